"""The mechanisms Sesuzen adds, each alone against the plain implementation's function for it: the layer norm, the
convolution over time with its carried rows, the placing of q, k, v with biases and the value norm, attention under
a window that keeps the first positions (keys planted just inside and just outside every edge so that a mask one
position off shows, in prompts and in single tokens, in every kernel that serves it), the delta rule with its
carried state, the norm and gate behind it, the gated experts; then the parts built from descriptions."""
import math

import pytest
import torch

import plain_sesuzen as P
from test_parts_gpu import Step, act, part, summed

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64
# on |got - ref| / (|ref| + mean |ref|), element by element: results stored in bfloat16 carry up to 2^-8 of their
# own size, and a product of bfloat16 inputs a few times that
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def bf(t):
    return t.to(torch.bfloat16).float()


def err(got, ref):
    ref = ref.to(torch.float64)
    d = (got.to(torch.float64).cpu() - ref).abs()
    return float((d / (ref.abs() + ref.abs().mean())).max())


def close(got, ref, dtype, what, roundings=1):
    assert torch.isfinite(got.float()).all(), f"{what}: not finite"
    e = err(got, ref)
    assert e < TOL[dtype] * roundings, f"{what}: error {e:.3e} ({dtype})"


# ---------------------------------------------------------------- layer norm
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,parts", [(56, 0), (104, 1), (1030, 3), (2048, 2)])
def test_layer_norm_with_the_pending_addition(dtype, H, parts):
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(H)
    T = 9
    resid = torch.randn(T, H, generator=g) * 3 + 1.5            # a mean that is not nought
    delta = torch.randn(parts, T, H, generator=g) if parts else None
    w, b = 1 + 0.3 * torch.randn(H, generator=g), 0.5 * torch.randn(H, generator=g)
    r = resid.clone().to(DEV)
    out = torch.zeros(T, H, dtype=DT[dtype], device=DEV)
    ops.add_layernorm(r, delta.to(DEV) if parts else None, w.to(DEV), b.to(DEV), 1e-5, out)
    v = resid + (delta.sum(0) if parts else 0)
    assert float((r.cpu() - v).abs().max()) < 1e-5               # the stream itself moves on
    close(out.cpu(), P.layer_norm(v.double(), w.double(), b.double(), 1e-5), dtype, "layer norm")
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    before = r.clone()
    few = torch.zeros(2, H, dtype=DT[dtype], device=DEV)
    ops.add_layernorm(r, None, w.to(DEV), None, 1e-5, few, rows)
    assert torch.equal(r, before)
    close(few.cpu(), P.layer_norm(v[[7, 2]].double(), w.double(), torch.zeros(H, dtype=torch.float64), 1e-5), dtype, "chosen rows, no bias")


# ---------------------------------------------------------------- convolution over time
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,C", [(4, 72), (2, 130), (1, 64), (8, 48), (3, 256)])
def test_convolution_over_time_in_portions(dtype, taps, C):
    """Three sequences brought in unequal portions (one token, two, fewer than the taps reach, many), in slots that
    are not in order; the rows carried between steps are the state."""
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(taps * C)
    tdt = DT[dtype]
    lens = [40, 7, 23]
    hs = [torch.randn(n, C, generator=g).to(tdt).float() for n in lens]
    w = (0.5 * torch.randn(C, taps, generator=g))
    refs = [P.time_conv(h.double(), w.double()) for h in hs]
    slots = [5, 0, 3]
    state = torch.zeros(6, max(taps - 1, 1), C, dtype=tdt, device=DEV)
    done = [0, 0, 0]
    got = [[], [], []]
    for portions in ([1, 2, 1], [2, 1, 9], [1, 1, 1], [30, 3, 5], [6, 0, 7]):
        seqs = [b for b in range(3) if portions[b] > 0]
        step = Step([portions[b] for b in seqs], [done[b] for b in seqs])
        step.keep["seq_slot"].copy_(torch.tensor([slots[b] for b in seqs], dtype=torch.int32))
        h = torch.cat([hs[b][done[b]:done[b] + portions[b]] for b in seqs]).to(tdt).to(DEV)
        out = torch.zeros_like(h)
        k = step.keep
        ops.causal_conv(h, out, w.to(DEV), state if taps > 1 else None, k["tok_seq"], k["tok_pos"], k["seq_start"], k["seq_past"],
                        k["seq_slot"], single_tokens=all(portions[b] == 1 for b in seqs))
        at = 0
        for b in seqs:
            got[b].append(out[at:at + portions[b]].cpu())
            at += portions[b]
            done[b] += portions[b]
    for b in range(3):
        assert done[b] == lens[b]
        close(torch.cat(got[b]), refs[b], dtype, f"convolution, sequence {b}")
    assert float(state[[1, 2, 4]].abs().max()) == 0              # other slots' state is not touched


# ---------------------------------------------------------------- placing q, k, v: biases and the value norm
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,extra", [(4, 2, 16, 16, 0), (3, 3, 24, 40, 5), (6, 2, 12, 8, 120), (2, 1, 128, 64, 8)])
def test_placing_with_biases_and_the_value_norm(dtype, H, G, d, dv, extra):
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * d)
    q_lens, past = [70, 1, 9], [0, 130, 60]
    step = Step(q_lens, past)
    T = sum(q_lens)
    width = H * d + G * d + G * dv + extra
    qkv = torch.randn(T, width, generator=g) * 3
    bias = torch.randn(width, generator=g)
    eps = 1e-3
    full = (qkv + bias).double()
    q_ref = full[:, :H * d].reshape(T, H, d)
    k_ref = full[:, H * d:H * d + G * d].reshape(T, G, d)
    v_ref = P.unit_rms(full[:, H * d + G * d:H * d + G * d + G * dv].reshape(T, G, dv), eps)
    tdt = DT[dtype]
    q_out = torch.zeros(T, H * d, dtype=tdt, device=DEV)
    kc = torch.zeros(step.n_pages, G, PAGE, d, dtype=tdt, device=DEV)
    vc = torch.zeros(step.n_pages, G, PAGE, dv, dtype=tdt, device=DEV)
    ops.kv_place(qkv.to(DEV), q_out, H, G, d, dv, bias.to(DEV), eps, step.keep["tok_seq"], step.keep["tok_pos"], step.table, kc, vc, PAGE)
    close(q_out.cpu().reshape(T, H, d), q_ref, dtype, "queries")
    seq, table, pos = step.keep["tok_seq"].cpu(), step.table.cpu(), step.keep["tok_pos"].cpu().long()
    for t in range(T):
        page, row = int(table[seq[t], pos[t] // PAGE]), int(pos[t] % PAGE)
        close(kc[page, :, row].cpu(), k_ref[t], dtype, f"key of token {t}")
        close(vc[page, :, row].cpu(), v_ref[t], dtype, f"value of token {t}")
    # no bias and no norm; the queries alone (a run that reads another run's cache)
    kc2 = torch.zeros_like(kc)
    ops.kv_place(qkv.to(DEV), q_out, H, G, d, dv, None, -1.0, step.keep["tok_seq"], step.keep["tok_pos"], step.table, kc2, vc, PAGE, write_cache=False)
    close(q_out.cpu(), qkv[:, :H * d].double(), dtype, "queries as they come")
    assert float(kc2.abs().max()) == 0


# ---------------------------------------------------------------- attention under a window that keeps the first positions
def planted_case(L, H, G, d, dv, window, sink, seed=0):
    """Queries all near one direction u.  Keys that lie along u with a large length, each outweighing all ordinary keys
    together: the last kept position (sink - 1) and the first one not kept (sink), so that a later query far away has
    to find the one and must not see the other; and every 37th position, so that queries pass, one after another,
    the places where such a key is the oldest one inside their window and the newest one outside."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(d, generator=g)
    u = u / u.norm()
    q = bf(u[None, None, :] * 4 + 0.3 * torch.randn(L, H, d, generator=g))
    k = 0.3 * torch.randn(L, G, d, generator=g)
    for p in range(L):
        if p % 37 == 36 or (sink and p in (sink - 1, sink)):
            k[p] = u * 6
    v = torch.randn(L, G, dv, generator=g)
    return q, bf(k), bf(v)


def paged(t, table_row, tdt, lo=0):
    """[L, G, w] -> cache [pages, G, 64, w] with logical page j of the sequence at table_row[j]; positions below
    ``lo`` are left out (pages that a window gave back hold nothing)."""
    L, G, w = t.shape
    cache = torch.zeros(int(max(table_row)) + 1, G, PAGE, w, dtype=tdt)
    for p in range(lo, L):
        cache[table_row[p // PAGE], :, p % PAGE] = t[p].to(tdt)
    return cache.to(DEV)


def windowed(q, k, v, scale, window, sink):
    return P.softmax_attention(q.double(), k.double(), v.double(), scale, P.window_mask(q.shape[0], window, sink))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,window,sink", [(2, 1, 16, 16, 7, 2), (3, 3, 24, 40, 50, 1), (4, 2, 12, 8, 64, 0), (2, 2, 64, 64, 100, 70),
                                                 (2, 1, 32, 32, 30, 5), (2, 1, 32, 32, None, 0)])
def test_generic_attention_window_and_kept_first_positions(dtype, H, G, d, dv, window, sink):
    from libllm_b200.csrc import ops
    L = 230
    q, k, v = planted_case(L, H, G, d, dv, window, sink)
    tdt = DT[dtype]
    table_row = [5, 2, 7, 0]
    kc, vc = paged(k, table_row, tdt), paged(v, table_row, tdt)
    i32 = dict(dtype=torch.int32, device=DEV)
    pos = torch.arange(L)
    ref = windowed(q, k, v, 0.4, window, sink)
    out = torch.zeros(L, H * dv, dtype=tdt, device=DEV)
    ops.attention_generic(q.reshape(L, H * d).to(tdt).to(DEV), out, kc, vc, torch.zeros(L, **i32), pos.to(**i32),
                          torch.tensor([table_row], **i32), H, G, d, PAGE, window, 0.4, v_head_dim=dv, sink=sink)
    close(out.cpu().reshape(L, H, dv), ref, dtype, "generic attention")
    if window:                         # what the planted keys are there for: an edge one off is far away
        assert err(windowed(q, k, v, 0.4, window + 1, sink), ref) > 0.2
        assert err(windowed(q, k, v, 0.4, window - 1, sink), ref) > 0.2
    if sink:
        assert err(windowed(q, k, v, 0.4, window, sink + 1), ref) > 0.2
        assert err(windowed(q, k, v, 0.4, window, sink - 1), ref) > 0.2


@pytest.mark.parametrize("d,H,G,window,sink", [(64, 4, 2, 100, 4), (128, 2, 1, 96, 70), (64, 2, 2, 64, 1), (128, 2, 2, 300, 3), (32, 4, 4, 50, 65),
                                               (96, 2, 1, 7, 2), (16, 2, 1, 33, 0), (64, 8, 2, 40, 130)])
def test_tiled_prompt_and_decode_attention_under_a_window_with_kept_first_positions(d, H, G, window, sink):
    """The bfloat16 kernels of prompt steps (tensor memory at head sizes 64 and 128; mma.sync at the others) and of
    single tokens against the plain attention: two sequences, one with tokens cached before the step; the pages
    between the kept first positions and the window hold nothing, as in a cache that gave them back."""
    from libllm_b200.csrc import ops
    tdt = torch.bfloat16
    L0, L1, past1 = 413, 300, 77
    i32 = dict(dtype=torch.int32, device=DEV)
    cases = [planted_case(L0, H, G, d, d, window, sink, 1), planted_case(L1, H, G, d, d, window, sink, 2)]
    rows0, rows1 = list(range(0, 8)), list(range(8, 13))
    kc = torch.cat([paged(cases[0][1], rows0, tdt), paged(cases[1][1], [r - 8 for r in rows1], tdt)])
    vc = torch.cat([paged(cases[0][2], rows0, tdt), paged(cases[1][2], [r - 8 for r in rows1], tdt)])
    table = torch.tensor([rows0, rows1 + [0] * 3], **i32)
    q = torch.cat([cases[0][0].reshape(L0, H * d), cases[1][0][past1:].reshape(L1 - past1, H * d)]).to(tdt).to(DEV)
    seq_start = torch.tensor([0, L0, L0 + L1 - past1], **i32)
    seq_past = torch.tensor([0, past1], **i32)
    refs = [windowed(c[0], c[1], c[2], 0.3, window, sink) for c in cases]
    ref = torch.cat([refs[0], refs[1][past1:]])
    T = q.shape[0]
    forms = [("mma", None)] + ([("tc", 0), ("tc", 1)] if d in (64, 128) else [])
    for kind, form in forms:
        out = torch.zeros(T, H * d, dtype=tdt, device=DEV)
        if kind == "mma":
            ops.attention_prefill(q, out, kc, vc, seq_start, seq_past, table, 2, L0, H, G, d, PAGE, window, 0.3, sink=sink)
        else:
            ops.attention_prefill_tc(q, out, kc, vc, seq_start, seq_past, table, 2, L0, H, G, d, PAGE, window, 0.3, form=form, sink=sink)
        torch.cuda.synchronize()
        close(out.cpu().reshape(T, H, d), ref, "bfloat16", f"prompt attention {kind} {form}")
    # single tokens, from a cache whose pages between the kept first positions and the window are gone (their
    # table entries are -1, as the cache leaves them): the last positions, and positions where a planted key is
    # the oldest inside the window and the newest outside it
    if d in (16, 32, 64, 128) and H // G in (1, 2, 3, 4, 8):
        for p0, p1 in ((L0 - 1, L1 - 1), (36 + 37 * 5 + window - 1, 36 + 37 * 3 + window), (sink + window - 1, sink + window)):
            p0, p1 = min(p0, L0 - 1), min(p1, L1 - 1)
            pos = torch.tensor([p0, p1], **i32)
            tab = table.clone()
            kept = (sink + PAGE - 1) // PAGE
            for b, p in ((0, p0), (1, p1)):
                first_needed = max(0, p + 1 - window + 1) // PAGE
                for j in range(kept, first_needed):
                    tab[b, j] = -1
            qd = torch.stack([cases[0][0][p0], cases[1][0][p1]]).reshape(2, H * d).to(tdt).to(DEV)
            want = torch.stack([refs[0][p0], refs[1][p1]])
            for n_splits, chunk in ((1, 512), (4, 128), (7, 64)):
                out = torch.zeros(2, H * d, dtype=tdt, device=DEV)
                ws_o = torch.zeros(2 * H * n_splits * d, device=DEV)
                ws_ml = torch.zeros(2 * H * n_splits * 2, device=DEV)
                ops.attention_decode(qd, out, kc, vc, pos, tab, H, G, d, PAGE, chunk, n_splits, window, 0.3, ws_o, ws_ml, sink=sink)
                close(out.cpu().reshape(2, H, d), want, "bfloat16", f"single-token attention at {p0}, {p1}, {n_splits} splits")


def test_a_kept_first_key_outweighs_the_whole_window():
    """The planted case: far behind the window the result is, to a few percent, the value at the last kept position."""
    q, k, v = planted_case(230, 2, 1, 32, 32, 20, 5)
    ref = windowed(q, k, v, 0.4, 20, 5)
    assert float((ref[210, 0] - v[4, 0].double()).abs().max()) < 0.1 * float(v[4, 0].abs().max())


# ---------------------------------------------------------------- the delta rule
def delta_inputs(T, H, d, rank, g):
    W = H * d
    proj = torch.randn(T, 5 * W + rank + 3, generator=g)          # r | k | v | g | a | low-rank input | padding
    return proj, torch.randn(W, rank, generator=g) * 0.7, torch.randn(W, generator=g) * 0.5, torch.randn(W, generator=g) * 0.5


def delta_reference(proj, w2, w0, ab, H, d, rank, S=None):
    T, W = proj.shape[0], H * d
    p = proj.double()
    r, k, v = (p[:, i * W:(i + 1) * W].reshape(T, H, d) for i in range(3))
    decay = torch.exp(-P.DECAY_SCALE * torch.sigmoid(torch.tanh(p[:, 5 * W:5 * W + rank]) @ w2.double().T + w0.double())).view(T, H, d)
    rate = torch.sigmoid(p[:, 4 * W:5 * W] + ab.double()).view(T, H, d)
    unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + P.KEY_EPS)
    return P.delta_scan(r, k, v, decay, rate, unit, S)


@pytest.mark.parametrize("H,d,rank", [(2, 16, 8), (3, 24, 5), (1, 128, 24), (5, 8, 3), (2, 64, 16), (1, 200, 9), (2, 32, 1)])
def test_delta_rule_with_carried_state(H, d, rank):
    """Two sequences in slots that are not in order, each brought in two steps (a long one and single tokens beside a
    prompt): the state written by one launch is what the next one starts from."""
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * d + rank)
    lens = [29, 11]
    data = [delta_inputs(n, H, d, rank, g) for n in lens]
    w2, w0, ab = data[0][1:]
    refs = [delta_reference(x[0], w2, w0, ab, H, d, rank) for x in data]
    W = H * d
    state = torch.zeros(4, H, d, d, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 1], **i32)
    got = [[], []]
    done = [0, 0]
    for portions in ([20, 1], [1, 1], [8, 9]):
        proj = torch.cat([data[b][0][done[b]:done[b] + portions[b]] for b in range(2)]).to(DEV)
        start = torch.tensor([0, portions[0], portions[0] + portions[1]], **i32)
        out = ops.delta_rule(proj, (0, W, 2 * W, 4 * W, 5 * W), rank, w2.to(DEV), w0.to(DEV), ab.to(DEV), P.DECAY_SCALE, P.KEY_EPS,
                             state, start, slots, H, d)
        got[0].append(out[:portions[0]].cpu())
        got[1].append(out[portions[0]:].cpu())
        for b in range(2):
            done[b] += portions[b]
    for b in range(2):
        ref_o, ref_S = refs[b]
        close(torch.cat(got[b]).reshape(lens[b], H, d), ref_o, "float32", f"delta rule, sequence {b}", roundings=5)
        # the state lies with a column's rows together: [slot, head, value, key]
        close(state[int(slots[b])].cpu().transpose(1, 2), ref_S, "float32", f"state of sequence {b}", roundings=5)
    assert float(state[[0, 2]].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dv", [(3, 24), (2, 64), (5, 8), (1, 200)])
def test_norm_per_head_weight_and_gate(dtype, H, dv):
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(H * dv)
    T = 13
    x, w, gate = torch.randn(T, H * dv, generator=g) * 4, 1 + 0.3 * torch.randn(H * dv, generator=g), torch.randn(T, H * dv + 7, generator=g)
    out = torch.zeros(T, H * dv, dtype=DT[dtype], device=DEV)
    ops.head_norm_gate(x.to(DEV), w.to(DEV), gate.to(DEV), 1e-5, H, dv, out)
    ref = P.unit_rms(x.double().view(T, H, dv), 1e-5).reshape(T, H * dv) * w.double() * torch.sigmoid(gate[:, :H * dv].double())
    close(out.cpu(), ref, dtype, "norm per head, weight, gate")
    ops.head_norm_gate(x.to(DEV), None, gate.to(DEV), -1.0, H, dv, out)
    close(out.cpu(), x.double() * torch.sigmoid(gate[:, :H * dv].double()), dtype, "the gate alone")


# ---------------------------------------------------------------- gated experts
@pytest.mark.parametrize("dtype,grouped", [("float32", False), ("bfloat16", False), ("bfloat16", True), ("bfloat16", "tc")])
@pytest.mark.parametrize("T,E,top,width,ff", [(37, 5, 2, 72, 24), (200, 8, 4, 128, 64), (3, 3, 3, 64, 40), (700, 4, 1, 64, 136)])
def test_gated_experts_with_the_choice_given(dtype, grouped, T, E, top, width, ff):
    """down(silu(gate x) * up x) of the chosen experts, the choice given (so that bfloat16 is compared on the products
    alone): rows on the CUDA cores, sorted tiles on mma.sync and on tcgen05."""
    from libllm_b200.csrc import ops
    g = torch.Generator().manual_seed(T + E)
    tdt = DT[dtype]
    x = torch.randn(T, width, generator=g).to(tdt)
    gate, up, down = (torch.randn(E, ff, width, generator=g) / math.sqrt(width)).to(tdt), (torch.randn(E, ff, width, generator=g) / math.sqrt(width)).to(tdt), \
        (torch.randn(E, width, ff, generator=g) / math.sqrt(ff)).to(tdt)
    chosen = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    weight = torch.softmax(torch.randn(T, top, generator=g), -1)
    stacked = torch.stack([gate, up], 2).reshape(E, 2 * ff, width).contiguous()      # rows 2n: gate, 2n + 1: up
    out = ops.moe_experts(x.to(DEV), stacked.to(DEV), down.to(DEV), chosen.to(DEV), weight.to(DEV), act="silu", weight_on="output",
                          grouped=grouped, gated=True)
    ref = torch.zeros(top, T, width, dtype=torch.float64)
    xd = x.double()
    for t in range(T):
        for c in range(top):
            e = int(chosen[t, c])
            a = xd[t] @ gate[e].double().T
            ref[c, t] = weight[t, c].double() * (((a * torch.sigmoid(a)) * (xd[t] @ up[e].double().T)) @ down[e].double().T)
    close(out.cpu(), ref, dtype, f"gated experts ({grouped})", roundings=2)


# ---------------------------------------------------------------- parts built from descriptions
def attention_tensors(H, nH, nKV, d, dv, g):
    r = lambda *s: bf(torch.randn(*s, generator=g) * 1.2 / math.sqrt(s[-1]) if len(s) > 1 else 0.5 * torch.randn(*s, generator=g))
    return {"m.q": r(nH * d, H), "m.q.b": r(nH * d), "m.k": r(nKV * d, H), "m.k.b": r(nKV * d), "m.v": r(nKV * dv, H), "m.v.b": r(nKV * dv),
            "m.g": r(nH * dv, H), "m.o": r(H, nH * dv)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,nH,nKV,d,dv,window,sink", [(72, 6, 2, 16, 16, 20, 3), (40, 5, 5, 32, 24, 70, 0), (64, 4, 1, 64, 64, 90, 66), (48, 2, 2, 24, 40, None, 0)])
def test_attention_part_prompt_then_single_tokens(dtype, H, nH, nKV, d, dv, window, sink):
    g = torch.Generator().manual_seed(H + d)
    w = attention_tensors(H, nH, nKV, d, dv, g)
    spec = dict(kind="attention", hidden=H, n_heads=nH, n_kv_heads=nKV, head_dim=d, v_head_dim=dv, scale=0.21, position=None, window=window,
                bias=True, q_bias="m.q.b", k_bias="m.k.b", v_bias="m.v.b", v_norm=dict(eps=1e-4), out_gate="m.g", q="m.q", k="m.k", v="m.v", o="m.o")
    if sink:
        spec["sink"] = sink
    mixer = part("mixer", spec, dtype)
    assert mixer.description["cache"]["kind"] == ("window" if window else "full") and mixer.description["cache"]["sink"] == (sink or None)
    assert (mixer.description["cache"]["k_dim"], mixer.description["cache"]["v_dim"]) == (d, dv)
    mixer.load(w)
    L, n_prompt = 150, 131
    x = bf(torch.randn(L, H, generator=g))
    m = dict(heads=nH, kv_heads=nKV, dim=d, vdim=dv, scale=0.21)
    if window:
        m["mask"] = dict(size=window, keep_first=sink)
    ref = P.attention_mixer(x.double(), {k: v.double() for k, v in w.items()}, "m.", m, 1e-4)
    tdt = DT[dtype]
    n_pages = 4
    kc = torch.zeros(n_pages, nKV, PAGE, d, dtype=tdt, device=DEV)
    vc = torch.zeros(n_pages, nKV, PAGE, dv, dtype=tdt, device=DEV)
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=DEV)
    cache = dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=n_pages, page_table=table.data_ptr(), table_width=4, page_size=PAGE)
    got, at = [], 0
    for n in [n_prompt] + [1] * (L - n_prompt):
        step = Step([n], [at])
        xs = x[at:at + n].to(tdt).to(DEV)
        out = mixer.forward(dict(step=step.json, x=act(xs), cache=cache))["out"]
        got.append(summed(out).cpu())
        at += n
    close(torch.cat(got), ref, dtype, "attention part", roundings=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,nH,d,rank", [(72, 3, 24, 5), (64, 2, 64, 16), (40, 5, 8, 8)])
def test_delta_part_prompt_then_single_tokens(dtype, H, nH, d, rank):
    g = torch.Generator().manual_seed(H + d)
    W = nH * d
    r = lambda *s: bf(torch.randn(*s, generator=g) * 1.2 / math.sqrt(s[-1]) if len(s) > 1 else 0.5 * torch.randn(*s, generator=g))
    w = {"m." + n: r(W, H) for n in ("r", "k", "v", "g", "a")}
    w.update({"m.a.b": r(W), "m.w1": r(rank, H), "m.w2": r(W, rank), "m.w0": r(W), "m.norm": bf(1 + 0.2 * torch.randn(W, generator=g)), "m.o": r(H, W)})
    spec = dict(kind="general_delta", hidden=H, n_heads=nH, head_dim=d, decay_rank=None, eps=1e-4, a_bias="m.a.b",
                **{n: "m." + n for n in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")})
    mixer = part("mixer", spec, dtype)
    assert mixer.description["cache"] is None
    assert mixer.description["state"] == [dict(name="general_delta.S", shape=[nH, d, d], dtype="float32")]
    assert [t["shape"] for t in mixer.description["tensor_needs"] if t["name"] == "m.w1"] == [[-1, H]]
    mixer.load(w)
    L, n_prompt = 60, 41
    x = bf(torch.randn(L, H, generator=g))
    wd = {k: v.double() for k, v in w.items()}
    survives = []
    ref = P.delta_mixer(x.double(), wd, "m.", dict(heads=nH, dim=d), 1e-4, survives)
    tdt = DT[dtype]
    state = torch.zeros(3, nH, d, d, device=DEV)
    st = [dict(name="general_delta.S", ptr=state.data_ptr(), shape=[nH, d, d], dtype="float32", n_slots=3)]
    got, at = [], 0
    for n in [n_prompt] + [1] * (L - n_prompt):
        step = Step([n], [at])
        step.keep["seq_slot"].fill_(2)
        xs = x[at:at + n].to(tdt).to(DEV)
        got.append(summed(mixer.forward(dict(step=step.json, x=act(xs), state=st))["out"]).cpu())
        at += n
    got = torch.cat(got)
    if dtype == "bfloat16":           # rows where a head all but cancels hang on the roundings of its inputs
        keep = survives[0] > 0.15
        got, ref = got[keep], ref[keep]
    close(got, ref, dtype, "delta part", roundings=3)
    assert float(state[:2].abs().max()) == 0 and float(state[2].abs().max()) > 0
