"""The mechanisms Sinezen adds, each alone against the plain implementation's function for it: the
norm of whole projections with the rotation and the cache append, attention with a block mask (keys
planted just inside and just outside every block so that a mask one position off shows), a gate per
head, values of another width, the choice of experts and the experts' products; then the parts
built from descriptions."""
import math

import pytest
import torch

import plain_sinezen as P
from test_parts_gpu import Step, act, part, summed

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64
# on |got - ref| / (|ref| + mean |ref|), element by element: results stored in bfloat16 carry up to 2^-8 of
# their own size, and a product of bfloat16 inputs a few times that
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def bf(t):
    return t.to(torch.bfloat16).float()


def err(got, ref):
    ref = ref.to(torch.float64)
    d = (got.to(torch.float64).cpu() - ref).abs()
    return float((d / (ref.abs() + ref.abs().mean())).max())


def close(got, ref, dtype, what, roundings=1):
    """``roundings``: 2 for a whole part, whose products round their inputs one after another."""
    assert torch.isfinite(got.float()).all(), f"{what}: not finite"
    e = err(got, ref)
    assert e < TOL[dtype] * roundings, f"{what}: error {e:.3e} ({dtype})"


def rope_table(n, dims, base):
    i = torch.arange(dims // 2, dtype=torch.float64)
    a = torch.arange(n, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    return torch.cat([a.cos(), a.sin()], 1).float().to(DEV)


# ---------------------------------------------------------------- norm + rotation + append
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,rot,extra", [(4, 2, 16, 16, 16, 0), (3, 3, 24, 40, 12, 5), (6, 2, 12, 8, 0, 2), (2, 1, 128, 64, 64, 8),
                                               (5, 5, 10, 6, 10, 1)])
def test_projection_norm_rotation_and_append(dtype, H, G, d, dv, rot, extra):
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * d)
    q_lens, past = [70, 1, 9], [0, 130, 60]
    step = Step(q_lens, past)
    T = sum(q_lens)
    width = H * d + G * d + G * dv + extra
    qkv = torch.randn(T, width, generator=g) * 3
    qn, kn = 1 + 0.3 * torch.randn(H * d, generator=g), 1 + 0.3 * torch.randn(G * d, generator=g)
    eps = 1e-3
    pos = step.keep["tok_pos"].cpu().long()
    q_ref = P.rms_norm(qkv[:, :H * d].double(), qn.double(), eps).reshape(T, H, d)
    k_ref = P.rms_norm(qkv[:, H * d:H * d + G * d].double(), kn.double(), eps).reshape(T, G, d)
    if rot:
        q_ref, k_ref = P.rotate(q_ref, pos, rot, 5e4), P.rotate(k_ref, pos, rot, 5e4)
    v_ref = qkv[:, H * d + G * d:H * d + G * d + G * dv].reshape(T, G, dv)
    tdt = DT[dtype]
    q_out = torch.zeros(T, H * d, dtype=tdt, device=DEV)
    kc = torch.zeros(step.n_pages, G, PAGE, d, dtype=tdt, device=DEV)
    vc = torch.zeros(step.n_pages, G, PAGE, dv, dtype=tdt, device=DEV)
    ops.qk_place(qkv.to(DEV), q_out, H, G, d, dv, qn.to(DEV), kn.to(DEV), eps, rope_table(256, rot, 5e4) if rot else None,
                 step.keep["tok_seq"], step.keep["tok_pos"], step.table, kc, vc, PAGE)
    close(q_out.cpu().reshape(T, H, d), q_ref, dtype, "queries")
    seq = step.keep["tok_seq"].cpu()
    table = step.table.cpu()
    for t in range(T):
        page, row = int(table[seq[t], pos[t] // PAGE]), int(pos[t] % PAGE)
        close(kc[page, :, row].cpu(), k_ref[t], dtype, f"key of token {t}")
        close(vc[page, :, row].cpu(), v_ref[t].double(), dtype, f"value of token {t}")
    # no norm, and the queries alone (a run that reads another run's cache)
    kc2 = torch.zeros_like(kc)
    ops.qk_place(qkv.to(DEV), q_out, H, G, d, dv, None, None, eps, rope_table(256, rot, 5e4) if rot else None,
                 step.keep["tok_seq"], step.keep["tok_pos"], step.table, kc2, vc, PAGE, write_cache=False)
    plain_q = qkv[:, :H * d].double().reshape(T, H, d)
    close(q_out.cpu().reshape(T, H, d), P.rotate(plain_q, pos, rot, 5e4) if rot else plain_q, dtype, "queries without a norm")
    assert float(kc2.abs().max()) == 0


# ---------------------------------------------------------------- attention under a block mask
def planted_case(L, H, G, d, dv, block, seed=0):
    """Queries all near one direction u; the keys at every block's first position and at the
    position before it lie along u with a large length, so that each of them outweighs all others
    together: a query sees its own block's first key and must not see the one before it.  Without
    a block it is the key at position 2 that stands out: every later query, hundreds of positions
    on, still has to find it."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(d, generator=g)
    u = u / u.norm()
    q = bf(u[None, None, :] * 4 + 0.3 * torch.randn(L, H, d, generator=g))
    k = 0.3 * torch.randn(L, G, d, generator=g)
    for p in range(L):
        if (block and (p % block == 0 or p % block == block - 1)) or (not block and p == 2):
            k[p] = u * 6
    v = torch.randn(L, G, dv, generator=g)
    return q, bf(k), bf(v)


def paged(t, table_row, tdt):
    """[L, G, w] -> cache [pages, G, 64, w] with logical page j of the sequence at table_row[j]."""
    L, G, w = t.shape
    cache = torch.zeros(int(max(table_row)) + 1, G, PAGE, w, dtype=tdt)
    for p in range(L):
        cache[table_row[p // PAGE], :, p % PAGE] = t[p].to(tdt)
    return cache.to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,block", [(2, 1, 16, 16, 7), (3, 3, 24, 40, 50), (4, 2, 12, 8, 64), (2, 2, 64, 64, 100), (2, 1, 32, 32, None)])
def test_generic_attention_block_mask_gate_and_value_width(dtype, H, G, d, dv, block):
    from libllm_b200.csrc import ops
    L = 230
    q, k, v = planted_case(L, H, G, d, dv, block)
    gate = torch.randn(L, H + 3, generator=torch.Generator().manual_seed(1))
    tdt = DT[dtype]
    table_row = [5, 2, 7, 0]
    kc, vc = paged(k, table_row, tdt), paged(v, table_row, tdt)
    i32 = dict(dtype=torch.int32, device=DEV)
    table = torch.tensor([table_row], **i32)
    pos = torch.arange(L)
    ref = P.attention_core(q, k, v, pos, pos, 0.4, block, gate[:, :H])
    out = torch.zeros(L, H * dv, dtype=tdt, device=DEV)
    ops.attention_generic(q.reshape(L, H * d).to(tdt).to(DEV), out, kc, vc, torch.zeros(L, **i32), pos.to(**i32), table, H, G, d, PAGE,
                          None, 0.4, v_head_dim=dv, block=block, gate=gate.to(DEV))
    close(out.cpu().reshape(L, H, dv), ref, dtype, "generic attention")
    if block:                          # what the planted keys are there for: a mask one off is far away
        wrong = P.attention_core(q, k, v, pos + 1, pos, 0.4, block, gate[:, :H])
        assert err(wrong, ref) > 0.2


@pytest.mark.parametrize("d,H,G,block", [(64, 4, 2, 100), (128, 2, 1, 96), (64, 2, 2, 64), (128, 2, 2, 300), (32, 4, 4, 50), (96, 2, 1, 7), (16, 2, 1, 33)])
def test_tiled_prompt_and_decode_attention_under_a_block_mask(d, H, G, block):
    """The bfloat16 kernels of prompt steps (tensor memory at head sizes 64 and 128, in both its
    forms; mma.sync at the others) and of single tokens against the plain attention: two sequences,
    one with tokens cached before the step, the step's portions starting inside a block."""
    from libllm_b200.csrc import ops
    tdt = torch.bfloat16
    L0, L1, past1 = 413, 300, 77
    i32 = dict(dtype=torch.int32, device=DEV)
    cases = [planted_case(L0, H, G, d, d, block, 1), planted_case(L1, H, G, d, d, block, 2)]
    rows0, rows1 = list(range(0, 8)), list(range(8, 13))
    kc = torch.cat([paged(cases[0][1], rows0, tdt), paged(cases[1][1], [r - 8 for r in rows1], tdt)])
    vc = torch.cat([paged(cases[0][2], rows0, tdt), paged(cases[1][2], [r - 8 for r in rows1], tdt)])
    table = torch.tensor([rows0, rows1 + [0] * 3], **i32)
    q = torch.cat([cases[0][0].reshape(L0, H * d), cases[1][0][past1:].reshape(L1 - past1, H * d)]).to(tdt).to(DEV)
    seq_start = torch.tensor([0, L0, L0 + L1 - past1], **i32)
    seq_past = torch.tensor([0, past1], **i32)
    refs = [P.attention_core(c[0], c[1], c[2], torch.arange(len(c[0])), torch.arange(len(c[0])), 0.3, block) for c in cases]
    ref = torch.cat([refs[0], refs[1][past1:]])
    T = q.shape[0]
    forms = [("mma", None)] + ([("tc", 1), ("tc", 2)] if d in (64, 128) else [])
    for kind, form in forms:
        out = torch.zeros(T, H * d, dtype=tdt, device=DEV)
        if kind == "mma":
            ops.attention_prefill(q, out, kc, vc, seq_start, seq_past, table, 2, L0, H, G, d, PAGE, None, 0.3, block=block)
        else:
            ops.attention_prefill_tc(q, out, kc, vc, seq_start, seq_past, table, 2, L0, H, G, d, PAGE, None, 0.3, form=form, block=block)
        torch.cuda.synchronize()
        close(out.cpu().reshape(T, H, d), ref, "bfloat16", f"prompt attention {kind} {form}")
    # single tokens: the last position of each sequence, and positions at a block's first and last place
    if d in (16, 32, 64, 128):
        first0, first1 = (L0 - 1) // block * block, (L1 - 1) // block * block      # where the sequences' last blocks begin
        for p0, p1 in ((L0 - 1, L1 - 1), (first0, max(0, first1 - 1)), (max(0, first0 - 1), first1)):
            pos = torch.tensor([p0, p1], **i32)
            qd = torch.stack([cases[0][0][p0], cases[1][0][p1]]).reshape(2, H * d).to(tdt).to(DEV)
            want = torch.stack([refs[0][p0], refs[1][p1]])
            for n_splits, chunk in ((1, 512), (4, 128)):
                out = torch.zeros(2, H * d, dtype=tdt, device=DEV)
                ws_o = torch.zeros(2 * H * n_splits * d, device=DEV)
                ws_ml = torch.zeros(2 * H * n_splits * 2, device=DEV)
                ops.attention_decode(qd, out, kc, vc, pos, table, H, G, d, PAGE, chunk, n_splits, None, 0.3, ws_o, ws_ml, block=block)
                close(out.cpu().reshape(2, H, d), want, "bfloat16", f"single-token attention at {p0}, {p1}, {n_splits} splits")


def test_a_far_key_outweighs_hundreds_of_near_ones():
    """The planted case without a block: the result at position 229 is, to a few percent, the value at position 2."""
    q, k, v = planted_case(230, 2, 1, 32, 32, None)
    pos = torch.arange(230)
    ref = P.attention_core(q, k, v, pos, pos, 0.4, None)
    assert float((ref[229, 0] - v[2, 0].double()).abs().max()) < 0.1 * float(v[2, 0].abs().max())


# ---------------------------------------------------------------- the stream beside the token rows
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("parts", [0, 1, 3])
def test_stream_beside_the_token_rows(dtype, parts):
    from libllm_b200.csrc import ops
    T, H = 37, 52
    g = torch.Generator().manual_seed(parts)
    resid, other = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    delta = torch.randn(parts, T, H, generator=g) if parts else None
    out = torch.zeros(T, 2 * H, dtype=DT[dtype], device=DEV)
    ops.concat_stream(resid.to(DEV), delta.to(DEV) if parts else None, other.to(DEV), out)
    want = torch.cat([resid + (delta.sum(0) if parts else 0), other], 1)
    close(out.cpu(), want.double(), dtype, "stream beside the token rows")


# ---------------------------------------------------------------- routed feed-forward
@pytest.mark.parametrize("E,top,score,renorm", [(5, 1, "sigmoid", False), (12, 3, "sigmoid", False), (40, 8, "softmax", True), (3, 3, "sigmoid", True)])
def test_choice_of_experts(E, top, score, renorm):
    from libllm_b200.csrc import ops
    z = torch.randn(50, E, generator=torch.Generator().manual_seed(E)) * 2
    chosen, weight = ops.moe_route(z.to(DEV), top, score, renorm)
    s = torch.sigmoid(z.double()) if score == "sigmoid" else torch.softmax(z.double(), -1)
    val, idx = torch.topk(s, top, dim=-1)
    if renorm:
        val = val / val.sum(-1, keepdim=True)
    assert torch.equal(chosen.cpu().long(), idx)
    assert float((weight.cpu().double() - val).abs().max()) < 1e-6
    if score == "sigmoid" and not renorm:
        idx2, val2 = P.route(torch.eye(E, dtype=torch.float64), z.double(), top)
        assert torch.equal(idx2, idx) and torch.equal(val2, val)


@pytest.mark.parametrize("dtype,grouped", [("float32", False), ("bfloat16", False), ("bfloat16", True), ("bfloat16", "tc")])
@pytest.mark.parametrize("T,E,top,width,ff", [(1, 4, 2, 64, 32), (37, 5, 1, 72, 24), (300, 3, 2, 48, 40), (150, 16, 3, 128, 136),
                                              (700, 6, 2, 256, 200)])
def test_experts_products(dtype, grouped, T, E, top, width, ff):
    """Rows by expert: more rows than a tile holds for one expert, experts that nobody chose, one row."""
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(T + E)
    x = bf(torch.randn(T, width, generator=g))
    up = bf(torch.randn(E, ff, width, generator=g) / math.sqrt(width))
    down = bf(torch.randn(E, width, ff, generator=g) / math.sqrt(ff))
    z = torch.randn(T, E, generator=g) * 2
    z[:, E - 1] = -30.0                                   # the last expert is never chosen
    if top < E - 1:
        z[: T // 2, 0] = 30.0                             # and the first one by half of the tokens
    chosen, weight = ops.moe_route(z.to(DEV), top, "sigmoid", False)
    tdt = DT[dtype]
    for weight_on in ("input", "output"):
        out = ops.moe_experts(x.to(tdt).to(DEV), up.to(tdt).to(DEV), down.to(tdt).to(DEV), chosen, weight, "gelu", weight_on, grouped)
        ref = torch.zeros(top, T, width, dtype=torch.float64)
        for t in range(T):
            for j in range(top):
                e, wt = int(chosen[t, j]), float(weight[t, j])
                w = {"up": up[e].double(), "down": down[e].double()}
                ref[j, t] = P.expert(w, "", wt * x[t:t + 1].double())[0] if weight_on == "input" else wt * P.expert(w, "", x[t:t + 1].double())[0]
        close(out.cpu(), ref, dtype, f"experts, weight on the {weight_on}")


# ---------------------------------------------------------------- parts from their descriptions
def mixer_weights(W, m, seed=0):
    g = torch.Generator().manual_seed(seed)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: bf(torch.randn(*s, generator=g) * 1.5 / math.sqrt(s[-1]))
    return {"l0.mix.q": r(H * d, W), "l0.mix.k": r(G * d, W), "l0.mix.v": r(G * dv, W), "l0.mix.o": r(W, H * dv), "l0.mix.g": r(H, W) * 2,
            "l0.mix.q.norm": bf(1 + 0.2 * torch.randn(H * d, generator=g)), "l0.mix.k.norm": bf(1 + 0.2 * torch.randn(G * d, generator=g))}


def mixer_spec(W, m, eps):
    pos = dict(kind="rope", head_dim=m["dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"], scaling=None) if m.get("rot") else None
    return dict(kind="attention", hidden=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                scale=m["scale"], block=m["mask"]["size"] if m.get("mask") else None, position=pos,
                qk_norm=dict(q="l0.mix.q.norm", k="l0.mix.k.norm", eps=eps), head_gate="l0.mix.g",
                q="l0.mix.q", k="l0.mix.k", v="l0.mix.v", o="l0.mix.o")


MIXERS = [dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.3, mask=dict(size=8), rot=dict(base=1e4, dims=8)),
          dict(heads=3, kv_heads=3, dim=24, vdim=40, scale=0.2, mask=dict(size=50), rot=dict(base=5e5, dims=24)),
          dict(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, mask=dict(size=70), rot=dict(base=1e4, dims=32)),
          dict(heads=2, kv_heads=2, dim=12, vdim=20, scale=0.3)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m", MIXERS, ids=lambda m: f"d{m['dim']}v{m['vdim']}")
def test_attention_part_with_every_option(dtype, m):
    """A prompt in one call, then tokens one by one, two sequences of unequal lengths sharing the
    calls, against the plain mixer over the whole sequences."""
    W, eps = 56, 1e-4
    tdt = DT[dtype]
    w = mixer_weights(W, m)
    mixer = part("mixer", mixer_spec(W, m, eps), dtype)
    mixer.load(w)
    need = mixer.description["cache"]
    block = m["mask"]["size"] if m.get("mask") else None
    assert (need["k_dim"], need["v_dim"], need["block"], need["kind"]) == (m["dim"], m["vdim"], block, "block" if block else "full")
    lens = [75, 9]
    n_single = 12
    g = torch.Generator().manual_seed(5)
    xs = [bf(torch.randn(n + n_single, W, generator=g)) for n in lens]
    refs = [P.attention_mixer(m, {k: v.double() for k, v in w.items()}, "l0.", x.double(), torch.arange(x.shape[0]), eps) for x in xs]
    kc = vc = None
    outs = [[], []]
    for i in range(n_single + 1):
        q_lens = lens if i == 0 else [1, 1]
        past = [0, 0] if i == 0 else [lens[0] + i - 1, lens[1] + i - 1]
        step = Step(q_lens, past)
        if kc is None:
            kc = torch.zeros(step.n_pages + 8, m["kv_heads"], PAGE, m["dim"], dtype=tdt, device=DEV)
            vc = torch.zeros(step.n_pages + 8, m["kv_heads"], PAGE, m["vdim"], dtype=tdt, device=DEV)
        x = torch.cat([xs[b][past[b]:past[b] + q_lens[b]] for b in range(2)]).to(tdt).to(DEV)
        out = summed(mixer.forward(dict(step=step.json, x=act(x),
                                        cache=dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=kc.shape[0],
                                                   page_table=step.table.data_ptr(), table_width=step.width, writes=True)))["out"])
        o = 0
        for b in range(2):
            outs[b].append(out[o:o + q_lens[b]].cpu())
            o += q_lens[b]
    for b in range(2):
        close(torch.cat(outs[b]), refs[b], dtype, f"attention part, sequence {b}", roundings=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act_name", ["gelu", "gelu_tanh", "silu"])
def test_mlp_part(dtype, act_name):
    T, H, I = 19, 40, 104
    g = torch.Generator().manual_seed(1)
    r = lambda *s: bf(torch.randn(*s, generator=g) / math.sqrt(s[-1]))
    w = {"f.up": r(I, H), "f.down": r(H, I)}
    ff = part("feed_forward", dict(kind="mlp", hidden=H, intermediate=I, activation=act_name, up="f.up", down="f.down"), dtype)
    ff.load(w)
    x = bf(torch.randn(T, H, generator=g))
    out = summed(ff.forward(dict(step=Step([T], [0]).json, x=act(x.to(DT[dtype]).to(DEV))))["out"])
    z = x.double() @ w["f.up"].double().T
    a = {"gelu": P.gelu_erf(z), "silu": z * torch.sigmoid(z),
         "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[act_name]
    close(out, a @ w["f.down"].double().T, dtype, f"mlp part {act_name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,shared", [(1, 4, 2, 24), (90, 6, 1, None), (70, 5, 3, 16)])
def test_routed_part(dtype, T, E, top, shared):
    H, I = 48, 32
    g = torch.Generator().manual_seed(T)
    r = lambda *s: bf(torch.randn(*s, generator=g) / math.sqrt(s[-1]))
    w = {"l0.mlp.router": r(E, H) * 6}
    for e in range(E):
        w[f"l0.mlp.e{e}.up"], w[f"l0.mlp.e{e}.down"] = r(I, H), r(H, I)
    spec = dict(kind="moe", hidden=H, experts=E, top=top, score="sigmoid", renormalize=False, weight_on="input", router="l0.mlp.router",
                expert=dict(intermediate=I, activation="gelu", up="l0.mlp.e{}.up", down="l0.mlp.e{}.down"), shared=None)
    mlp = dict(kind="moe", router=dict(experts=E, top=top), expert=dict(ff=I))
    if shared:
        w["l0.mlp.shared.up"], w["l0.mlp.shared.down"] = r(shared, H), r(H, shared)
        spec["shared"] = dict(kind="mlp", hidden=H, intermediate=shared, activation="gelu", up="l0.mlp.shared.up", down="l0.mlp.shared.down")
        mlp["shared"] = dict(ff=shared)
    ff = part("feed_forward", spec, dtype)
    assert sorted(n["name"] for n in ff.description["tensor_needs"]) == sorted(w)
    ff.load(w)
    x = bf(torch.randn(T, H, generator=g))
    ref = P.moe_ff(mlp, {k: v.double() for k, v in w.items()}, "l0.", x.double())
    out = summed(ff.forward(dict(step=Step([T], [0]).json, x=act(x.to(DT[dtype]).to(DEV))))["out"])
    # a choice between two experts that hangs on the input's last bits is no test: such rows are left out
    s = torch.sigmoid(x.double() @ w["l0.mlp.router"].double().T).sort(-1, descending=True).values
    clear = (s[:, top - 1] - s[:, top]) > 1e-2 if top < E else torch.ones(T, dtype=torch.bool)
    assert int(clear.sum()) >= T * 0.5
    close(out[clear], ref[clear], dtype, "routed part")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("with_ff", [True, False])
def test_parallel_block_alone(dtype, with_ff):
    """x + mixer(norm x) + ff(norm x) from its description: the pending addition it is handed is
    applied first, and what it leaves pending completes the sum."""
    W, eps = 56, 2e-5
    m = MIXERS[1]
    tdt = DT[dtype]
    g = torch.Generator().manual_seed(2)
    r = lambda *s: bf(torch.randn(*s, generator=g) / math.sqrt(s[-1]))
    w = mixer_weights(W, m, seed=4)
    w["l0.norm1"] = bf(1 + 0.1 * torch.randn(W, generator=g))
    spec = dict(kind="parallel", norm=dict(kind="rmsnorm", size=W, eps=eps, weight="l0.norm1"), mixer=mixer_spec(W, m, eps), ff=None)
    c = dict(width=W, norm=dict(eps=eps), layers=[dict(type="attention", mixer=m, mlp=None)])
    if with_ff:
        w.update({"l0.mlp.gate": r(72, W), "l0.mlp.up": r(72, W), "l0.mlp.down": r(W, 72)})
        spec["ff"] = dict(kind="swiglu", hidden=W, intermediate=72, gate="l0.mlp.gate", up="l0.mlp.up", down="l0.mlp.down")
        c["layers"][0]["mlp"] = dict(kind="dense", ff=72)
    block = part("block", spec, dtype)
    assert sorted(n["name"] for n in block.description["tensor_needs"]) == sorted(w)
    block.load(w)
    T = 60
    step = Step([T], [0])
    kc = torch.zeros(step.n_pages, m["kv_heads"], PAGE, m["dim"], dtype=tdt, device=DEV)
    vc = torch.zeros(step.n_pages, m["kv_heads"], PAGE, m["vdim"], dtype=tdt, device=DEV)
    x0, pend = torch.randn(T, W, generator=g), 0.5 * torch.randn(T, W, generator=g)
    resid = x0.to(DEV).clone()
    pending = pend.to(DEV)
    out = block.forward(dict(step=step.json, hidden=W, resid=resid.data_ptr(), pending=act(pending),
                             cache=dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=kc.shape[0], page_table=step.table.data_ptr(),
                                        table_width=step.width, writes=True)))
    got = resid.cpu() + (summed(out["pending"]).cpu() if out["pending"] is not None else 0)
    ref = P.layer(c, {k: v.double() for k, v in w.items()}, 0, (x0 + pend).double(), torch.arange(T))
    close(got, ref, dtype, "parallel block", roundings=2)
