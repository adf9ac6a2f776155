"""Small Sinezen configurations and random weights for the tests, made here (not by the library),
and the comparison rules."""
from __future__ import annotations

import math
from typing import Dict, List

import torch


def attn(heads, kv, dim, vdim, mask, rot_dims, base=10000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.0 / math.sqrt(dim))
    if mask:
        m["mask"] = dict(size=mask)
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims)
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, shared=None):
    d = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def layer(mixer, mlp):
    return dict(type="attention", mixer=mixer, mlp=mlp)


# Z1: keys as wide as values in a multiple of 16 (the tiled kernels), a mask much shorter than a page, every
#     layer inside the loop.
# Z2: sizes that are no multiple of 8 or 16, values wider and narrower than keys, a layer without a
#     feed-forward, masks that are no divisor of the page, layers before and after the loop, experts
#     without a shared one, one and several kv heads per group.
# Z3: no loop at all, heads of 64 (the tensor-memory prompt kernel), a partial rotation, a mask longer
#     than any test sequence in one layer and one of 96 in the other, three experts of eight.
# Z4: one repetition of a loop (the input mix still applies), a rotation of all and of no channels.
# Z5: widths that are multiples of 2 only (no 16-byte rows anywhere), a negative score scale.
# Z6: no routed layer, heads of 64 and of 32 with values as wide as keys (the tiled kernels in prompt and
#     single-token steps): in bfloat16 every position has to lie inside the bound.
CONFIGS: Dict[str, dict] = {
    "Z1": dict(architecture="Sinezen", vocab=200, width=64, norm=dict(eps=1e-6),
               layers=[layer(attn(4, 2, 16, 16, 8, 8), dense(96)),
                       layer(attn(4, 2, 16, 16, 24, 16, base=3e4, scale=0.2), moe(4, 2, 32, shared=48))],
               loop=dict(start=0, stop=2, times=2)),
    "Z2": dict(architecture="Sinezen", vocab=131, width=72, norm=dict(eps=1e-5),
               layers=[layer(attn(3, 3, 24, 40, 50, 12, base=5e5, scale=0.3), None),
                       layer(attn(6, 2, 12, 8, 7, 12), moe(5, 1, 24)),
                       layer(attn(2, 1, 36, 36, 100, 36, base=777.0), dense(80))],
               loop=dict(start=1, stop=2, times=3)),
    "Z3": dict(architecture="Sinezen", vocab=300, width=128, norm=dict(eps=2e-6),
               layers=[layer(attn(2, 2, 64, 64, 4096, 32), dense(160)),
                       layer(attn(4, 1, 64, 64, 96, 64, scale=0.11), moe(8, 3, 40, shared=64))]),
    "Z4": dict(architecture="Sinezen", vocab=97, width=48, norm=dict(eps=1e-5),
               layers=[layer(attn(2, 1, 32, 32, 33, 32), dense(64)),
                       layer(attn(3, 3, 16, 24, None, None), moe(3, 3, 16, shared=16))],
               loop=dict(start=1, stop=2, times=1)),
    "Z5": dict(architecture="Sinezen", vocab=77, width=50, norm=dict(eps=1e-5),
               layers=[layer(attn(5, 5, 10, 6, 9, 6, scale=0.4), moe(3, 2, 22, shared=14)),
                       layer(attn(3, 1, 18, 18, 20, 10, scale=-0.2), dense(34))],
               loop=dict(start=0, stop=1, times=2)),
    "Z6": dict(architecture="Sinezen", vocab=180, width=96, norm=dict(eps=1e-5),
               layers=[layer(attn(2, 1, 64, 64, 72, 32), dense(128)),
                       layer(attn(4, 2, 32, 32, 40, 32, base=2e4, scale=0.15), None),
                       layer(attn(3, 3, 48, 48, 500, 16), dense(72))],
               loop=dict(start=1, stop=3, times=2)),
}


def is_routed(c: dict) -> bool:
    return any(L["mlp"] and L["mlp"]["kind"] == "moe" for L in c["layers"])


def tensor_shapes(c: dict) -> Dict[str, List[int]]:
    W = c["width"]
    out = {"embed": [c["vocab"], W], "final.norm": [W], "head": [c["vocab"], W]}
    if c.get("loop"):
        out["loop.in"] = [W, 2 * W]
    for i, L in enumerate(c["layers"]):
        m, p = L["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": [W], p + "mix.q": [H * d, W], p + "mix.k": [G * d, W], p + "mix.v": [G * dv, W],
                    p + "mix.q.norm": [H * d], p + "mix.k.norm": [G * d], p + "mix.g": [H, W], p + "mix.o": [W, H * dv]})
        f = L["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": [f["ff"], W], p + "mlp.up": [f["ff"], W], p + "mlp.down": [W, f["ff"]]})
        else:
            out[p + "mlp.router"] = [f["router"]["experts"], W]
            for e in range(f["router"]["experts"]):
                out[f"{p}mlp.e{e}.up"] = [f["expert"]["ff"], W]
                out[f"{p}mlp.e{e}.down"] = [W, f["expert"]["ff"]]
            if f.get("shared"):
                out[p + "mlp.shared.up"] = [f["shared"]["ff"], W]
                out[p + "mlp.shared.down"] = [W, f["shared"]["ff"]]
    return out


def random_weights(c: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bfloat16-representable float32 tensors: matrices ~ N(0, 1/fan_in) times a factor that keeps
    the stream of order one, norm weights around 1, router rows large enough that the choice of
    experts seldom hangs on the last bits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        if len(shape) == 1:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g) * 4.0 / math.sqrt(shape[1])
        elif name.endswith("mix.g"):
            t = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[1])
        else:
            t = torch.randn(shape, generator=g) * 1.5 / math.sqrt(shape[1])
        out[name] = t.to(torch.bfloat16).float()
    return out


def tokens(c: dict, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, c["vocab"], (n,), generator=g).tolist()


def row_errors(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per position: the root mean square of the difference over the vocabulary, relative to the
    root mean square of the reference's logits (over everything)."""
    ref = ref.to(torch.float64)
    d = got.to(torch.float64).cpu() - ref
    return (d * d).mean(-1).sqrt() / (ref * ref).mean().sqrt()


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits at every product's input; and a
# rounding may now and then turn a close choice between two experts, which changes that position
# by far more than rounding (float32 shows that the choice itself is right): so one position in ten
# may lie outside, and the median must lie well inside.
TOL = {"float32": 2e-5, "bfloat16": 5e-2}


def check_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, routed: bool = True) -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    e = row_errors(got, ref)
    if dtype == "float32" or not routed:
        assert float(e.max()) < TOL[dtype], f"{what}: row error {float(e.max()):.3e} at position {int(e.argmax())} ({dtype})"
        return
    over = int((e > TOL[dtype]).sum())
    assert over <= max(2, e.numel() // 10), f"{what}: {over} of {e.numel()} positions beyond {TOL[dtype]} ({dtype})"
    assert float(e.median()) < TOL[dtype] / 3, f"{what}: median row error {float(e.median()):.3e} ({dtype})"
