"""A plain, slow implementation of the Sesuzen decoder in float64, one function per mechanism.

It shares no code with the library: it reads the same config.json keys and tensor names and
computes every position of one sequence at once with dense matrices and explicit loops.  The
tests compare the library's logits, and single mechanisms, against it.

Layout of a model (config.json): ``vocab``, ``width``, ``max_positions``, ``norm.eps``,
``canon.taps``, ``logit_softcap``, ``layers`` (entry i: ``type`` "attention" or "general_delta",
``mixer`` with its sizes, ``mlp`` null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "router":
{experts, top}, "expert": {ff}}``; tensors ``l<i>.*``) and ``loop`` {start, stop, times}: layers
start .. stop-1 run ``times`` times in a row with the same weights.  A layer is
x += mixer(mix_in(ln1 x)); x += ff(ln2 x).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64
DECAY_SCALE = math.exp(-0.5)      # the decay of the delta rule is exp(-DECAY_SCALE * sigmoid(.))
KEY_EPS = 1e-6                    # under the root of the unit key's length


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w + b over the last axis."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by sqrt(mean(x^2) + eps) over the last axis, no weight."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def time_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps] -> h + conv(h): out[t] = h[t] + sum_j w[:, j] h[t - (taps - 1) + j], rows before
    the first counting as zero (the last tap lies on the token itself)."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * h[s]
    return out


def window_mask(n: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[n, n] true where query i sees key j: j <= i, and j among the last ``size`` positions up to i or among
    the first ``keep_first`` of the sequence.  ``size`` None: every earlier key."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    near = (i - j < size) if size else torch.ones(n, n, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, visible: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; head h reads key/value head h // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=F)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        out[:, head] = torch.softmax(s.masked_fill(~visible, -math.inf), dim=-1) @ v[:, g]
    return out


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Projections with biases, no rotation, values normalised per head, windowed softmax with kept first
    tokens, a sigmoid gate per channel from the same input, output projection."""
    T, H, G, d = h.shape[0], m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", d)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = unit_rms((h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv), eps)
    mask = m.get("mask")
    visible = window_mask(T, mask["size"] if mask else None, mask.get("keep_first", 0) if mask else 0)
    o = softmax_attention(q, k, v, m["scale"], visible).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def delta_vectors(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, H: int, d: int):
    """What each token brings to the recurrence: r, k, v, decay, removal rate, unit key, all [T, H, d]."""
    T = h.shape[0]
    r, k, v = ((h @ w[p + n].T).view(T, H, d) for n in ("r", "k", "v"))
    decay = torch.exp(-DECAY_SCALE * torch.sigmoid(torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, d)
    unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + KEY_EPS)
    return r, k, v, decay, rate, unit


def delta_scan(r, k, v, decay, rate, unit, S: Optional[torch.Tensor] = None, cancelled: Optional[torch.Tensor] = None):
    """S [H, d, d] (keys x values), token by token:  S <- decay * S - (rate * unit) (unit^T S) + k v^T, both terms
    from the old S; o = S^T r.  Returns (o [T, H, d], the last S).  ``cancelled`` [T, H] receives |o| / | |S|^T |r| |:
    how much of the sum's terms is left in the result (the norm that follows blows a nearly cancelled head's
    rounding up; at the first token o = v (k.r), whose sign hangs on k.r)."""
    T, H, d = r.shape
    S = torch.zeros(H, d, d, dtype=F) if S is None else S.clone()
    out = torch.zeros(T, H, d, dtype=F)
    for t in range(T):
        for hd in range(H):
            old = S[hd]
            seen = unit[t, hd] @ old                                          # [d values]
            S[hd] = decay[t, hd][:, None] * old - torch.outer(rate[t, hd] * unit[t, hd], seen) + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S[hd].T @ r[t, hd]
            if cancelled is not None:
                cancelled[t, hd] = out[t, hd].norm() / (S[hd].abs().T @ r[t, hd].abs()).norm().clamp_min(1e-300)
    return out, S


def delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, survives: Optional[list] = None) -> torch.Tensor:
    """``survives`` collects, per token, the smallest share of a head's sum that survives cancellation."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    cancelled = torch.ones(T, H, dtype=F) if survives is not None else None
    o, _ = delta_scan(*delta_vectors(h, w, p, H, d), cancelled=cancelled)
    if survives is not None:
        survives.append(cancelled.min(dim=1).values)
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """down(relu(up h)^2)"""
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def route(z: torch.Tensor, top: int):
    """z [T, E] -> (chosen [T, top], weights [T, top]): the largest logits (the lower index on ties) and the
    softmax over the chosen logits alone."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict, margins: Optional[list] = None) -> torch.Tensor:
    """Sum over the chosen experts of weight * down(silu(gate h) * up h).  ``margins`` collects, per token, by how
    much the last chosen logit beats the best one left out (a choice that hangs on less than rounding is no test)."""
    z = h @ w[p + "router"].T
    chosen, weight = route(z, f["router"]["top"])
    if margins is not None and f["router"]["top"] < z.shape[1]:
        ranked = torch.sort(z, dim=-1, descending=True).values
        margins.append(ranked[:, f["router"]["top"] - 1] - ranked[:, f["router"]["top"]])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(chosen.shape[1]):
            e = p + f"e{int(chosen[t, c])}."
            g = h[t] @ w[e + "gate"].T
            out[t] += weight[t, c] * (((g * torch.sigmoid(g)) * (h[t] @ w[e + "up"].T)) @ w[e + "down"].T)
    return out


def layer_runs(c: dict) -> List[int]:
    n, loop = len(c["layers"]), c.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def forward(c: dict, w: Dict[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None,
            margins: Optional[list] = None, survives: Optional[list] = None) -> torch.Tensor:
    """Logits at every position of one sequence, [T, vocab], float64.  ``margins`` and ``survives``: see routed_ff and
    delta_mixer (how far each position is from hanging on a rounding)."""
    w = {k: v.to(F) for k, v in w.items()}
    eps, T = c["norm"]["eps"], len(tokens)
    x = w["embed"][torch.tensor(tokens)] + w["pos"][:T]
    for i in layer_runs(c):
        L, p = c["layers"][i], f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if c.get("canon"):
            h = time_conv(h, w[p + "canon1"])
        if L["type"] == "attention":
            x = x + attention_mixer(h, w, p + "mix.", L["mixer"], eps)
        else:
            x = x + delta_mixer(h, w, p + "mix.", L["mixer"], eps, survives)
        if L["mlp"] is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + (dense_ff(h, w, p + "mlp.") if L["mlp"]["kind"] == "dense" else routed_ff(h, w, p + "mlp.", L["mlp"], margins))
        if streams is not None:
            streams.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T
    cap = c.get("logit_softcap", 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits
