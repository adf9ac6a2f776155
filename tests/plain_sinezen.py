"""A plain, slow implementation of the Sinezen decoder in float64, one function per mechanism.

It shares no code with the library: it reads the same config.json keys and tensor names and
computes every position of one sequence at once with dense matrices.  The tests compare the
library's logits, and single parts, against it.

Layout of a model (config.json):

* ``layers``: a list; entry i has ``type`` (the mixer, here ``attention``), ``mixer`` (its sizes)
  and ``mlp`` (``{"kind": "dense", "ff"}``, ``{"kind": "moe", "router": {experts, top},
  "expert": {ff}, "shared": {ff} or absent}`` or null); its tensors are named ``l<i>.*``.
* ``loop`` {start, stop, times}: the layers from ``start`` up to, not including, ``stop`` are
  repeated ``times`` times and share their weights; a repetition begins by replacing the stream
  with ``W_in [x; x0]`` (tensor ``loop.in``), x0 being the token embedding.
* a layer is parallel: with h = rmsnorm(x), x <- x + mixer(h) + ff(h).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` channels of every head are rotated, channel i paired
    with i + dims/2, by the angle pos * base^(-2i/dims); the other channels pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    ang = pos.to(F)[:, None] * base ** (-2.0 * i / dims)[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_mask(q_pos: torch.Tensor, k_pos: torch.Tensor, size: int) -> torch.Tensor:
    """[Tq, Tk] true where key j is visible to query i: j <= i and both in the same block of
    ``size`` positions counted from position 0."""
    qi, kj = q_pos[:, None], k_pos[None, :]
    return (kj <= qi) & (torch.div(qi, size, rounding_mode="floor") == torch.div(kj, size, rounding_mode="floor"))


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, k_pos: torch.Tensor, scale: float,
                   block: Optional[int], gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv] -> [Tq, H, dv]: softmax over the visible keys of
    scale * q.k, head h reading kv head h // (H / G); ``gate`` [Tq, H] multiplies by its sigmoid."""
    H, G = q.shape[1], k.shape[1]
    visible = chunk_mask(q_pos, k_pos, block if block else 1 << 40)
    out = torch.zeros(q.shape[0], H, v.shape[2], dtype=F)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head].to(F) @ k[:, g].to(F).T) * scale
        a = torch.softmax(s.masked_fill(~visible, -math.inf), dim=-1)
        out[:, head] = a @ v[:, g].to(F)
        if gate is not None:
            out[:, head] *= torch.sigmoid(gate[:, head:head + 1].to(F))
    return out


def attention_mixer(m: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor, pos: torch.Tensor, eps: float) -> torch.Tensor:
    """The attention mixer on the normalised input h [T, width] of positions pos [T]."""
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", d)
    T = h.shape[0]
    q = h @ w[p + "mix.q"].T
    k = h @ w[p + "mix.k"].T
    v = h @ w[p + "mix.v"].T
    # one norm over the whole projection, before the heads are split and before the rotation
    q = rms_norm(q, w[p + "mix.q.norm"], eps)
    k = rms_norm(k, w[p + "mix.k.norm"], eps)
    q, k = q.reshape(T, H, d), k.reshape(T, G, d)
    if m.get("rot"):
        q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"])
    v = v.reshape(T, G, dv)
    # without a mask entry every earlier key is visible
    out = attention_core(q, k, v, pos, pos, m["scale"], m["mask"]["size"] if m.get("mask") else None, h @ w[p + "mix.g"].T)
    return out.reshape(T, H * dv) @ w[p + "mix.o"].T


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    a = h @ w[p + "mlp.gate"].T
    return ((a * torch.sigmoid(a)) * (h @ w[p + "mlp.up"].T)) @ w[p + "mlp.down"].T


def expert(w: Dict[str, torch.Tensor], p: str, x: torch.Tensor) -> torch.Tensor:
    return gelu_erf(x @ w[p + "up"].T) @ w[p + "down"].T


def route(w_router: torch.Tensor, h: torch.Tensor, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top]): scores are sigmoid(router h), the top
    ones are taken, and the weights are those scores as they are."""
    s = torch.sigmoid(h @ w_router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def moe_ff(mlp: dict, w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    idx, val = route(w[p + "mlp.router"], h, mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w[p + "mlp.e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            # the weight scales the expert's input, not its output
            out[t] += expert(w, f"{p}mlp.e{e}.", val[t, j] * h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + expert(w, p + "mlp.shared.", h)
    return out


def feed_forward(mlp: Optional[dict], w, p: str, h: torch.Tensor) -> Optional[torch.Tensor]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return dense_ff(w, p, h)
    if mlp["kind"] == "moe":
        return moe_ff(mlp, w, p, h)
    raise ValueError(mlp["kind"])


def layer_runs(c: dict) -> List[Tuple[int, bool]]:
    """(layer, whether a pass of the loop starts right before it), in running order."""
    n = len(c["layers"])
    loop = c.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    runs += [(i, False) for i in range(b, n)]
    return runs


def layer(c: dict, w, i: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    L = c["layers"][i]
    p = f"l{i}."
    eps = c["norm"]["eps"]
    h = rms_norm(x, w[p + "norm1"], eps)
    if L["type"] != "attention":
        raise ValueError(L["type"])
    y = attention_mixer(L["mixer"], w, p, h, pos, eps)
    f = feed_forward(L.get("mlp"), w, p, h)
    return x + (y if f is None else y + f)


def forward(c: dict, w: Dict[str, torch.Tensor], tokens, want_streams: bool = False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer run)."""
    w = {k: v.to(F) for k, v in w.items()}
    pos = torch.arange(len(tokens))
    x0 = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    x = x0
    streams = []
    for i, starts_pass in layer_runs(c):
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(c, w, i, x, pos)
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], c["norm"]["eps"]) @ w["head"].T
    return (logits, torch.stack(streams)) if want_streams else logits
