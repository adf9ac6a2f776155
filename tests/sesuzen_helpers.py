"""Small Sesuzen configurations and random weights for the tests, made here (not by the library),
and the comparison rules."""
from __future__ import annotations

import math
from typing import Dict, List

import torch


def attn(heads, kv, dim, vdim, size, keep, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.0 / math.sqrt(dim))
    if size:
        m["mask"] = dict(size=size, keep_first=keep)
    return dict(type="attention", mixer=m)


def delta(heads, dim, rank=None):
    m = dict(heads=heads, dim=dim)
    if rank:
        m["rank"] = rank              # else the rank is what "mix.w1" is stored with (RANKS below)
    return dict(type="general_delta", mixer=m)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))


def layer(mixer, mlp):
    return dict(mlp=mlp, **mixer)


def config(vocab, width, eps, taps, cap, layers, loop=None, max_positions=512):
    c = dict(architecture="Sesuzen", vocab=vocab, width=width, max_positions=max_positions, norm=dict(eps=eps), canon=dict(taps=taps),
             logit_softcap=cap, layers=layers)
    if loop:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return c


# S1: every layer inside the loop; a window much shorter than a page that keeps three first tokens.
# S2: sizes that are no multiple of 8 or 16, values wider and narrower than keys, a layer without a feed-forward,
#     one expert of five, kept first tokens 0 and 1, layers before and after the loop, two taps.
# S3: no loop, heads of 64 (the tiled kernels), a window longer than a page, delta heads of 64.
# S4: one tap (no state of the convolution), more kept first tokens than a page holds, a window longer than
#     any test sequence, a loop that runs once, all experts chosen, delta heads of 128 and a rank of 24.
# S5: five taps, delta heads of 8 and of 32, full attention without a mask, an empty loop.
# S6: no routed layer: in bfloat16 whole sequences are compared.
# S7: widths that are multiples of 2 only (no 16-byte rows anywhere), delta heads of 10 with a rank of 3, two key/value
#     heads for six query heads of 18 with values of 6, six taps, a cap that binds (logits beyond it).
CONFIGS: Dict[str, dict] = {
    "S1": config(150, 64, 1e-6, 3, 20.0,
                 [layer(delta(2, 16), dense(96)), layer(attn(4, 2, 16, 16, 24, 3, scale=0.2), moe(4, 2, 32))], loop=(0, 2, 2)),
    "S2": config(131, 72, 1e-5, 2, 30.0,
                 [layer(attn(3, 3, 24, 40, 50, 1, scale=0.3), None), layer(delta(3, 24), moe(5, 1, 24)),
                  layer(attn(6, 2, 12, 8, 7, 0), dense(80))], loop=(1, 2, 3)),
    "S3": config(300, 128, 2e-6, 4, 50.0,
                 [layer(attn(4, 1, 64, 64, 80, 5, scale=0.11), moe(8, 3, 40)), layer(delta(2, 64), dense(160)),
                  layer(attn(2, 2, 64, 64, 200, 2), dense(96))]),
    "S4": config(97, 48, 1e-5, 1, 15.0,
                 [layer(attn(2, 1, 32, 32, 10, 70), dense(64)), layer(delta(1, 128, rank=24), moe(3, 3, 16)),
                  layer(attn(3, 3, 16, 24, 4096, 2), None)], loop=(1, 2, 1)),
    "S5": config(77, 56, 1e-5, 5, 25.0,
                 [layer(delta(5, 8), moe(3, 2, 22)), layer(attn(2, 1, 20, 12, None, 0, scale=0.4), dense(34)),
                  layer(delta(2, 32), dense(40))], loop=(1, 1, 4)),
    "S6": config(180, 96, 1e-5, 4, 30.0,
                 [layer(attn(2, 1, 64, 64, 72, 4), dense(128)), layer(delta(3, 32), dense(72)),
                  layer(attn(4, 2, 32, 32, 40, 9, scale=0.15), None), layer(delta(2, 48), dense(64))], loop=(1, 3, 2)),
    "S7": config(90, 50, 3e-6, 6, 4.0,
                 [layer(delta(3, 10), dense(34)), layer(attn(6, 2, 18, 6, 21, 2, scale=0.25), moe(3, 2, 22)),
                  layer(delta(1, 22), None)], loop=(0, 2, 2)),
}
# the rank of the decay's low-rank input where the configuration does not give it: read from the tensor
RANKS = {"S1": 8, "S2": 5, "S3": 16, "S4": 24, "S5": 12, "S6": 7, "S7": 3}


def is_routed(c: dict) -> bool:
    return any(L["mlp"] and L["mlp"]["kind"] == "moe" for L in c["layers"])


def tensor_shapes(c: dict, rank: int) -> Dict[str, List[int]]:
    W = c["width"]
    out = {"embed": [c["vocab"], W], "pos": [c["max_positions"], W], "final.norm": [W], "final.norm.b": [W]}
    for i, L in enumerate(c["layers"]):
        m, p = L["mixer"], f"l{i}."
        out.update({p + "norm1": [W], p + "norm1.b": [W], p + "canon1": [W, c["canon"]["taps"]]})
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": [H * d, W], p + "mix.q.b": [H * d], p + "mix.k": [G * d, W], p + "mix.k.b": [G * d],
                        p + "mix.v": [G * dv, W], p + "mix.v.b": [G * dv], p + "mix.g": [H * dv, W], p + "mix.o": [W, H * dv]})
        else:
            N, r = m["heads"] * m["dim"], m.get("rank", rank)
            out.update({p + "mix." + n: [N, W] for n in ("r", "k", "v", "g", "a")})
            out.update({p + "mix.a.b": [N], p + "mix.w1": [r, W], p + "mix.w2": [N, r], p + "mix.w0": [N], p + "mix.norm": [N],
                        p + "mix.o": [W, N]})
        f = L["mlp"]
        if f is None:
            continue
        out.update({p + "norm2": [W], p + "norm2.b": [W]})
        if f["kind"] == "dense":
            out.update({p + "mlp.up": [f["ff"], W], p + "mlp.down": [W, f["ff"]]})
        else:
            out[p + "mlp.router"] = [f["router"]["experts"], W]
            for e in range(f["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": [f["expert"]["ff"], W], f"{p}mlp.e{e}.up": [f["expert"]["ff"], W],
                            f"{p}mlp.e{e}.down": [W, f["expert"]["ff"]]})
    return out


def random_weights(c: dict, seed: int = 0, rank: int = 8) -> Dict[str, torch.Tensor]:
    """bfloat16-representable float32 tensors: matrices ~ N(0, 1/fan_in) times a factor that keeps the stream of order
    one, norm weights around 1 and biases around 0, position vectors as large as token rows, router rows large enough
    that the choice of experts seldom hangs on the last bits, decays spread between fast and slow."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c, rank).items():
        r = lambda *s: torch.randn(*s, generator=g)
        if name.endswith(".b") or name.endswith("w0"):
            t = 0.5 * r(shape)
        elif name.endswith("canon1"):
            t = 0.4 * r(shape)
        elif len(shape) == 1:
            t = 1.0 + 0.2 * r(shape)
        elif name in ("embed", "pos"):
            t = r(shape) * (1.0 if name == "embed" else 0.5)
        elif name.endswith("router"):
            t = r(shape) * 4.0 / math.sqrt(shape[1])
        elif name.endswith("w2"):
            t = r(shape) * 2.0 / math.sqrt(shape[1])
        elif name.endswith("mix.g") or name.endswith("mix.a"):
            t = r(shape) * 2.0 / math.sqrt(shape[1])
        else:
            t = r(shape) * 1.3 / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16).float()
    return out


def tokens(c: dict, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(9000 + seed)
    return torch.randint(0, c["vocab"], (n,), generator=g).tolist()


def row_errors(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: the root mean square of the difference over the vocabulary, relative to the root mean square
    of the reference's logits (over everything)."""
    ref = ref.to(torch.float64)
    d = got.to(torch.float64).cpu() - ref
    return (d * d).mean(-1).sqrt() / (ref * ref).mean().sqrt()


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits at every product's input.  Two things make a
# position hang on such roundings, and neither is a test of anything (float32 shows the computation itself to be right):
# * a choice between two experts whose router logits lie closer than the rounding's own size: the token then runs
#   through another expert, and every later position sees that through the cache and the state;
# * a head of the delta rule whose sum cancels to a small share of its terms (at a first token, where the head's
#   result is v (k.r), when k.r is nearly nought: then even its sign): the norm behind it divides by what is left.
# So in bfloat16 a sequence is compared up to its first close call or head that all but vanishes (``clear``: the number
# of leading positions before it) and must be finite after, and a position where less than 0.15 of a head survives
# gets that much more room (``slack``).
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
CLOSE_CALL = 0.12                 # router logits are of order 4; their bfloat16 error of order 0.02
VANISHES = 0.01                   # share of a head's terms


def clear_rows(margins: list, survives: list, n: int) -> int:
    """The number of leading positions before the first one that hangs on a rounding (``margins``, ``survives`` as
    plain_sesuzen.forward collects them)."""
    first = n
    for m, limit in [(x, CLOSE_CALL) for x in margins] + [(x, VANISHES) for x in survives]:
        close = (m < limit).nonzero()
        if close.numel():
            first = min(first, int(close[0]))
    return first


def slack_rows(survives: list, n: int) -> torch.Tensor:
    out = torch.ones(n, dtype=torch.float64)
    for m in survives:
        out = torch.maximum(out, (0.15 / m.clamp_min(VANISHES)).clamp(1.0, 6.0))
    return out


def check_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, routed: bool = True, clear: int = None,
               slack: torch.Tensor = None) -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    e = row_errors(got, ref)
    if dtype == "bfloat16" and slack is not None:
        e = e / slack
    if dtype == "bfloat16" and clear is not None:
        e = e[:clear]
        if e.numel() == 0:
            return
    assert float(e.max()) < TOL[dtype], f"{what}: row error {float(e.max()):.3e} at position {int(e.argmax())} of {e.numel()} compared ({dtype})"
