"""Bonolorn in the engine against the plain implementation: every mechanism alone, then the whole model under every
way of cutting the work, with pages and state slots that are freed and used again, and generation through the entry
point (GPU)."""
import math
from types import SimpleNamespace

import pytest
import torch

import bonolorn_util as bz
import plain_bonolorn as plain
import replay_util as ru

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"


def stream():
    return torch.cuda.current_stream().cuda_stream


def batch_of(q_lens, slots, starts=None):
    """What the kernels read of a step: token -> sequence map, first token of each sequence, slots, positions."""
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    seq = [i for i, n in enumerate(q_lens) for _ in range(n)]
    starts = starts or [0] * len(q_lens)
    pos = [s + j for s, n in zip(starts, q_lens) for j in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(num_tokens=cu[-1], num_seqs=len(q_lens), token_seq=i32(seq), cu_tokens=i32(cu), state_slots=i32(slots),
                           positions=i32(pos), q_lens=list(q_lens), start_positions=list(starts), max_q_len=max(q_lens),
                           max_context_len=max(s + n for s, n in zip(starts, q_lens)), span_hint=0, plans={})


# ---- each mechanism alone --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("hidden", [40, 72, 256, 1000, 4096, 5120])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_plain_and_behind_a_sublayer(hidden, dtype):
    from lucciola_b200 import ops
    T = 6
    r = torch.randn(T, hidden, device=DEV) * 3 + 20.0            # far from zero: the mean must be taken off before squaring
    a, b = (torch.randn(T, hidden, device=DEV).to(dtype) * 2 + 1 for _ in range(2))
    w = 1 + 0.3 * torch.randn(hidden, device=DEV)
    rows = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    out = torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops.layernorm(out, r, w, 1e-5, stream(), rows=rows)
    want = plain.layer_norm(r.double().cpu()[[4, 0, 2]], w.double().cpu(), 1e-5)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    for pair in ((a, b), (a, None)):
        res, copy = r.clone(), torch.empty(T, hidden, dtype=dtype, device=DEV)
        ops.layernorm_add(res, pair[0], pair[1], 0.6, 0.9, w, 0.3, 1e-5, stream(), copy=copy)
        v = 0.6 * a.double() + (0.9 * b.double() if pair[1] is not None else 0)
        want = r.double().cpu() + 0.3 * plain.layer_norm(v.cpu(), w.double().cpu(), 1e-5)
        assert (res.double().cpu() - want).abs().max() <= 3e-6 * want.abs().max()          # the stream is 32-bit whatever the type
        assert torch.equal(copy, res.to(dtype))


@pytest.mark.parametrize("width", [8, 41, 320])
def test_sinusoidal_positions_far_out(width):
    from lucciola_b200 import ops
    table = torch.randn(30, width, device=DEV).to(torch.bfloat16)
    ids = torch.tensor([3, 29, 0, 3, 7], dtype=torch.int32, device=DEV)
    at = torch.tensor([0, 1, 1125, 70001, 999999], dtype=torch.int32, device=DEV)
    freq = (10000.0 ** (-2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)).to(DEV)
    x = torch.empty(5, width, device=DEV)
    ops.embedding(x, ids, table, stream(), positions=at, sin_freq=freq)
    want = table[ids.long()].double().cpu() + plain.sinusoid_positions(at.cpu(), width)[:, :width]
    assert (x.double().cpu() - want).abs().max() <= 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act,limit", [("gelu_tanh", 0.0), ("clamped_swish", 1.5), ("clamped_swish", 0.4)])
def test_gate_activations(dtype, act, limit):
    from lucciola_b200 import ops
    T, inter, K = 9, 128, 64
    gu = (torch.randn(T, 2 * inter, device=DEV) * 2).to(dtype)
    out = torch.empty(T, inter, dtype=dtype, device=DEV)
    ops.swiglu(out, gu[:, :inter], gu[:, inter:], stream(), act=act, limit=limit)

    def ref(g, u):
        if act == "gelu_tanh":
            return plain.gelu_tanh(g) * u
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1)
    want = ref(gu[:, :inter].double(), gu[:, inter:].double())
    assert (out.double() - want).abs().max() <= (2e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()
    if dtype == torch.bfloat16:                        # the same inside the tensor-core product's epilogue, few tokens and many
        for M in (3, 200, 1100):
            x = torch.randn(M, K, device=DEV).to(dtype)
            gate, up = (torch.randn(inter, K, device=DEV).to(dtype) * 0.3 for _ in range(2))
            o = torch.empty(M, inter, dtype=dtype, device=DEV)
            ops.gemm_tcgen05(o, x, ops.interleave_gate_up(gate, up), stream(), swiglu=True, act=act, limit=limit)
            want = ref(x.double() @ gate.double().T, x.double() @ up.double().T)
            assert (o.double() - want).abs().max() <= 1e-2 * want.abs().max(), M


@pytest.mark.parametrize("side", [0, 1, 2, 4])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 20, 40), (1, 40, 40), (3, 36, 12), (2, 128, 64), (4, 64, 128), (6, 8, 8), (1, 200, 33), (1, 300, 40), (2, 4, 8), (1, 256, 32)])
def test_decay_recurrence_alone(heads, dim, vdim, side):
    """Two sequences in unequal portions (single tokens, a few, many), against the plain recurrence with identity maps;
    a row of the state that belongs to another request stays as it is.  Token by token, and with the outputs of 16
    tokens formed side by side, the rows of the state whole or shared out over two or four CTAs."""
    from lucciola_b200 import ops
    n, m = heads * dim, heads * vdim
    W = 2 * n + 2 * m
    lens_total, slots = (37, 5), [1, 3]
    pre = [torch.randn(t, W + 3, device=DEV)[:, 3:] for t in lens_total]                 # a column range of a wider matrix
    decay = torch.tensor(([0.9, 1.0, 0.5, 0.999, 0.97, 0.3] * 2)[:heads], device=DEV)
    norm_w = 1 + 0.2 * torch.randn(m, device=DEV)
    state = torch.zeros(5, heads, dim, vdim, device=DEV)
    state[2] = float("nan")
    got, at = [[], []], [0, 0]
    for sizes in ([1, 2], [17, 1], [3, 1], [16, 1], [0, 0]):
        live = [i for i in range(2) if at[i] < lens_total[i] and sizes[i]]
        if not live:
            continue
        lens = [min(sizes[i], lens_total[i] - at[i]) for i in live]
        x = torch.cat([pre[i][at[i]:at[i] + k] for i, k in zip(live, lens)])
        x = torch.cat([torch.zeros(x.shape[0], 1, device=DEV), x], dim=1)[:, 1:]         # row-strided
        step = batch_of(lens, [slots[i] for i in live])
        few = max(lens) if max(lens) <= 3 else 0
        split = (side if few == 0 else 0) and max(1, min(side, dim // 32), -(-dim // 256))     # into how many shares the rows are cut
        o = torch.empty((split, x.shape[0], m) if split else (x.shape[0], m), device=DEV)
        before = state.clone()
        ops.decay_recurrence(x, 0, n, 2 * n, decay, state, o, step, heads, dim, vdim, stream(), max_tokens_a_seq=few, row_split=split)
        if split:                                                              # the other kernel from the same state: the same state after
            st2, o2 = before.clone(), torch.empty(x.shape[0], m, device=DEV)
            ops.decay_recurrence(x, 0, n, 2 * n, decay, st2, o2, step, heads, dim, vdim, stream())
            live_rows = [slots[i] for i in live]
            assert (st2[live_rows] - state[live_rows]).abs().max() <= 1e-5 * st2[live_rows].abs().max()
            assert (o2 - o.sum(0)).abs().max() <= 1e-5 * o2.abs().max()
        out = torch.empty(x.shape[0], m + 2, device=DEV)[:, 2:]
        ops.rmsnorm_gated(out, o, norm_w, x[:, 2 * n + m:], 0.7, 1e-5, stream())
        k0 = 0
        for i, k in zip(live, lens):
            got[i].append(out[k0:k0 + k]); k0 += k; at[i] += k
    assert at == list(lens_total)
    eye = torch.eye(W, dtype=torch.float64)
    w = {"q": eye[:n], "k": eye[n:2 * n], "v": eye[2 * n:2 * n + m], "g": eye[2 * n + m:], "norm": norm_w.double().cpu(),
         "o": torch.eye(m, dtype=torch.float64)}
    for i in range(2):
        want, S = plain.decay_attention(pre[i].double().cpu(), w, heads, dim, vdim, decay.double().cpu(), 1e-5)
        g = torch.cat(got[i]).double().cpu()
        assert (g - 0.7 * want).abs().max() <= 2e-5 * want.abs().max(), i
        assert (state[slots[i]].double().cpu() - S).abs().max() <= 1e-5 * S.abs().max()
    assert torch.isnan(state[2]).all() and torch.equal(state[0], torch.zeros_like(state[0]))


def paged(total, page, heads, dim, fill):
    """Block tables in scrambled order and a pool whose unused pages hold NaN, from per-sequence tensors [n, heads, dim]."""
    max_pages = max(-(-t // page) for t in total)
    perm = torch.randperm(len(total) * max_pages + 5).tolist()
    table = torch.full((len(total), max_pages), -1, dtype=torch.int32)
    pool = torch.full((len(total) * max_pages + 5, heads, page, dim), float("nan"))
    for s, x in enumerate(fill):
        for i in range(-(-total[s] // page)):
            table[s, i] = perm.pop()
            chunk = x[i * page:(i + 1) * page]                                         # [n, heads, dim]
            pool[table[s, i], :, :chunk.shape[0]] = chunk.transpose(0, 1)
    return table, pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,page,window", [(3, 1, 20, 12, 8, 24), (4, 2, 64, 64, 16, 40), (8, 2, 128, 128, 16, 300), (2, 2, 32, 80, 4, 7),
                                                           (4, 4, 64, 64, 16, 0), (1, 1, 40, 40, 8, 1), (16, 4, 128, 128, 32, 96), (6, 3, 8, 8, 16, 33)])
def test_a_query_finds_its_one_key_inside_the_window_and_not_outside(dtype, heads, kv, dim, vdim, page, window):
    """Every head of every query is made to point at one key (itself, the one before, the last the window lets in, the
    first it shuts out, keys at and beside page borders) with a score far above the others.  Where the key is inside
    the window the result must be that key's value; where it is outside, or far back, the plain function over the
    same numbers says what comes out instead.  A prompt's portion behind a cached part, a whole prompt and a decoded
    token in one batch; pages in scrambled order, every other page NaN; the distance bias on."""
    from lucciola_b200 import ops
    from lucciola_b200.parts import BatchShape, GatedBiasAttention, PlanView, Runtime, distance_slopes
    starts, lens = [300, 0, 517], [77, 130, 1]
    total = [s + n for s, n in zip(starts, lens)]
    unit = lambda n, d: torch.nn.functional.normalize(torch.randn(n, kv, d), dim=-1).mul(d ** 0.5).to(dtype).float()
    keys, vals = [unit(t, dim) for t in total], [torch.randn(t, kv, vdim).to(dtype).float() for t in total]
    table, kpool = paged(total, page, kv, dim, keys)
    vpool = torch.full((kpool.shape[0], kv, page, vdim), float("nan"))
    for s in range(3):
        for i in range(-(-total[s] // page)):
            chunk = vals[s][i * page:(i + 1) * page]
            vpool[table[s, i], :, :chunk.shape[0]] = chunk.transpose(0, 1)
    step = batch_of(lens, [0, 1, 2], starts)
    step.block_tables = [table.to(DEV)]
    T, per = sum(lens), heads // kv
    w_eff = window if window > 0 else 10 ** 9
    slopes = torch.tensor(distance_slopes(heads), dtype=torch.float64)
    q = torch.zeros(T, heads, dim)
    want = torch.zeros(T, heads, vdim, dtype=torch.float64)
    t = 0
    for s in range(3):
        for j in range(lens[s]):
            p = starts[s] + j
            picks = [p, max(p - 1, 0), max(p - w_eff + 1, 0), max(p - w_eff, 0), (p // page) * page, max((p // page) * page - 1, 0), p // 2, 0,
                     max(p - w_eff + 2, 0), max(p - w_eff - 1, 0)]
            picks = [min(x, p) for x in picks]
            for h in range(heads):
                key = picks[(t + h) % len(picks)]
                c = keys[s][key, h // per]
                q[t, h] = c * (600.0 / c.pow(2).sum())            # its own score 600 (less the distance bias), another key's 600 x the cosine
                lo = max(0, p - w_eff + 1)
                sc = keys[s][lo:p + 1, h // per].double() @ q[t, h].to(dtype).double() - slopes[h] * (p - torch.arange(lo, p + 1)).double()
                want[t, h] = torch.softmax(sc, 0) @ vals[s][lo:p + 1, h // per].double()
                if lo <= key:
                    assert (want[t, h] - vals[s][key, h // per].double()).abs().max() < 1e-3 * vals[s].abs().max()
            t += 1
    part = GatedBiasAttention(Runtime(DEV, dtype), "x", 8, heads, kv, dim, vdim, 1.0, window, 1e-6, distance_slopes(heads))
    plan = part.plan(BatchShape(lens, starts, max(lens), max(total), max(total))) if part.plan_key() is not None else None
    view = PlanView({k: torch.tensor(v, device=DEV) for k, v in plan.arrays.items()}, plan.host) if plan is not None else None
    q, kpool, vpool = q.to(dtype).to(DEV), kpool.to(dtype).to(DEV), vpool.to(dtype).to(DEV)
    out = torch.empty(T, heads, vdim, dtype=dtype, device=DEV)
    ops.attention(q, out, kpool, vpool, step, 0, heads, kv, dim, page, window, 1.0, stream(), plan=view, v_dim=vdim,
                  slopes=slopes.float().to(DEV))
    err = (out.double().cpu() - want).abs().max().item()
    assert err <= (2e-2 if dtype == torch.bfloat16 else 1e-4) * want.abs().max().item(), err
    # single tokens alone (the kernels of decoding): the last token of each sequence
    dec = batch_of([1, 1, 1], [0, 1, 2], [t - 1 for t in total])
    dec.block_tables = step.block_tables
    rows = [lens[0] - 1, lens[0] + lens[1] - 1, T - 1]
    plan1 = part.plan(BatchShape([1, 1, 1], dec.start_positions, 1, max(total), max(total))) if plan is not None else None
    view1 = PlanView({k: torch.tensor(v, device=DEV) for k, v in plan1.arrays.items()}, plan1.host) if plan1 is not None else None
    q1, out1 = q[rows].contiguous(), torch.empty(3, heads, vdim, dtype=dtype, device=DEV)
    ops.attention(q1, out1, kpool, vpool, dec, 0, heads, kv, dim, page, window, 1.0, stream(), plan=view1, v_dim=vdim,
                  slopes=slopes.float().to(DEV))
    assert (out1.double().cpu() - want[rows]).abs().max().item() <= (2e-2 if dtype == torch.bfloat16 else 1e-4) * want.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_store_of_heads_with_values_of_another_size(dtype):
    """Queries and keys normed per head from the 32-bit columns of a wider product, keys and values into their pages
    (values with rows of their own size), the gate of one number a head."""
    from lucciola_b200 import ops
    H, G, d, dv, page = 4, 2, 20, 12, 4
    lens, starts = [3, 1, 6], [0, 9, 2]
    step = batch_of(lens, [0, 1, 2], starts)
    T = sum(lens)
    n1, n2, n3 = H * d, H * d + G * d, H * d + G * d + G * dv
    pre = torch.randn(T, n3 + H + 5, device=DEV) * 2
    qw, kw = 1 + 0.2 * torch.randn(d, device=DEV), 1 + 0.2 * torch.randn(d, device=DEV)
    table = torch.tensor([[5, -1, -1], [0, 1, 7], [2, 3, -1]], dtype=torch.int32, device=DEV)
    kp = torch.full((8, G, page, d), 99.0, dtype=dtype, device=DEV)
    vp = torch.full((8, G, page, dv), 99.0, dtype=dtype, device=DEV)
    q = torch.empty(T, H, d, dtype=dtype, device=DEV)
    ops.rope_kv(pre[:, :n1], pre[:, n1:n2], pre[:, n2:n3], q, step.positions, H, G, d, 1e-6, stream(), q_norm_w=qw, k_norm_w=kw,
                k_cache=kp, v_cache=vp, token_seq=step.token_seq, block_table=table, page_size=page, v_dim=dv)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    P = pre.double().cpu()
    want_q = plain.rms_norm(P[:, :n1].reshape(T, H, d), qw.double().cpu(), 1e-6)
    want_k = plain.rms_norm(P[:, n1:n2].reshape(T, G, d), kw.double().cpu(), 1e-6)
    want_v = P[:, n2:n3].reshape(T, G, dv)
    assert (q.double().cpu() - want_q).abs().max() <= tol * want_q.abs().max()
    written = set()
    for t in range(T):
        s, p = int(step.token_seq[t]), int(step.positions[t])
        pg = int(table[s, p // page])
        written.add((pg, p % page))
        assert (kp[pg, :, p % page].double().cpu() - want_k[t]).abs().max() <= tol * want_k.abs().max(), t
        assert (vp[pg, :, p % page].double().cpu() - want_v[t]).abs().max() <= tol * want_v.abs().max(), t
    for pg in range(8):
        for sl in range(page):
            if (pg, sl) not in written:
                assert (kp[pg, :, sl] == 99.0).all() and (vp[pg, :, sl] == 99.0).all()
    heads = torch.randn(T, H, dv, device=DEV).to(dtype)
    out = torch.empty(T, H * dv + 8, dtype=dtype, device=DEV)[:, 8:]
    ops.head_gate(out, heads, pre[:, n3:n3 + H], 0.6, stream())
    want = heads.double().cpu() * torch.sigmoid(P[:, n3:n3 + H])[:, :, None] * 0.6
    assert (out.double().cpu().view(T, H, dv) - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 3, 2), (6, 2, 3, 2), (2, 1, 2, 1), (8, 2, 1, 1), (16, 4, 2, 1), (64, 8, 8, 4), (5, 5, 5, 5),
                                                     (256, 8, 8, 4), (9, 1, 9, 3)])
def test_router_against_the_plain_choice(experts, top, groups, keep):
    from lucciola_b200 import ops
    T = 300
    z = torch.randn(T, experts + 3, device=DEV)[:, 3:] * 2
    corr = torch.randn(experts, device=DEV) * 0.5 - 0.6               # many choice scores below zero
    ids, wts = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    ops.route_topk(ids, wts, z, corr, groups, keep, 1.7, stream())
    chosen, weights = plain.route(z.double().cpu(), torch.eye(experts, dtype=torch.float64), corr.double().cpu(), top, groups, keep, 1.7)
    # a choice that hangs on the last bits of a 32-bit score may differ; everywhere else the sets and the weights agree
    s = torch.sigmoid(z.double().cpu()) + corr.double().cpu()
    same = 0
    for t in range(T):
        a, b = ids[t].cpu().tolist(), chosen[t].tolist()
        if sorted(a) != sorted(b):
            gap = (s[t][sorted(set(a) ^ set(b))]).diff().abs().min().item()
            assert gap < 1e-5, (t, a, b)
            continue
        same += 1
        assert len(set(a)) == top
        got = dict(zip(a, wts[t].cpu().tolist()))
        for e, x in zip(b, weights[t].tolist()):
            assert abs(got[e] - x) <= 1e-5 * max(1.0, abs(x))
    assert same >= T - 3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,experts,top,ff", [(1, 40, 2, 1, 32), (7, 72, 6, 2, 24), (70, 256, 8, 2, 128), (300, 64, 16, 4, 64), (33, 128, 5, 5, 100), (1000, 96, 64, 6, 16),
                                                (2000, 128, 4, 2, 128), (1500, 256, 16, 4, 64), (777, 64, 3, 3, 192)])
def test_routed_experts_against_the_plain_sum(dtype, T, W, experts, top, ff):
    """The whole part (router, lists by expert, both products, weighted sum, the expert for every token) with weights of
    its own; in bfloat16 the corrections are spread so that rounding cannot change a choice.  The last sizes have so many
    tokens an expert that the bfloat16 engine pads the experts' runs to tiles and takes the tensor-memory product."""
    from lucciola_b200.parts import GatedFeedForward, RoutedExperts, Runtime
    rt = Runtime(DEV, dtype)
    rt.stream = stream()
    limit = 1.3
    shared = GatedFeedForward(rt, "m.shared.gate", "m.shared.up", "m.shared.down", W, 48, act="clamped_swish", limit=0.9)
    part = RoutedExperts(rt, "m", W, experts, top, ff, "clamped_swish", limit, 1.5, groups=1, keep=1, shared=shared)
    g = torch.Generator().manual_seed(T + W)
    w = {s.name: (torch.randn(*s.shape, generator=g) * (1.5 / s.shape[-1] ** 0.5)).to(torch.bfloat16) for s in part.all_param_specs()}
    w["m.correction"] = (torch.randperm(experts, generator=g).float() * 3.0).to(torch.bfloat16) if dtype == torch.bfloat16 else w["m.correction"]
    part.bind_all(lambda name: w[name].to(DEV).to(dtype))
    h = torch.randn(T, W, generator=g).to(torch.bfloat16)
    out = part.forward(h.to(DEV).to(dtype), None)
    wd = {k[2:]: v.double() for k, v in w.items()}
    mlp = {"router": {"top": top, "groups": {"count": 1, "keep": 1}, "scale": 1.5}, "expert": {"limit": limit}, "shared": {"limit": 0.9}}
    want = plain.expert_feed_forward(h.double(), wd, mlp)
    err = (out.double().cpu() - want).abs().max().item()
    assert err <= (2e-5 if dtype == torch.float32 else 2e-2) * want.abs().max().item(), err


# ---- the whole model -------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder).  Beside each configuration X: "Xd" with routing that does not hang on a
    score's last bits (for bfloat16), and "Asharp" / "Csharp" whose attention picks out single keys (and "d" of those)."""
    out = {}
    for name, cfg in bz.CONFIGS.items():
        for suffix, kw in (("", {}), ("d", dict(decisive=True))):
            w = bz.make_weights(cfg, 100 + len(out), **kw)
            out[name + suffix] = (cfg, w, bz.write_model(tmp_path_factory.mktemp(f"bonolorn_{name}{suffix}"), cfg, w))
    for base in ("A", "C"):
        for suffix, kw in (("sharp", dict(sharp=4.0)), ("sharpd", dict(sharp=4.0, decisive=True))):
            cfg = bz.CONFIGS[base]
            w = bz.make_weights(cfg, 200 + len(out), **kw)
            out[base + suffix] = (cfg, w, bz.write_model(tmp_path_factory.mktemp(f"bonolorn_{base}{suffix}"), cfg, w))
    return out


def pick(name, dtype):
    """The weights a comparison in this type uses."""
    return name + "d" if dtype == "bfloat16" else name


def make_runner(models, name, dtype, num_pages, graphs=False, slots=4, **kw):
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    page = bz.PAGE[name[0]]
    return build_runner(models[name][2], EngineOptions(dtype=dtype, block_size=page, max_blocks=num_pages, max_num_seqs=slots,
                                                       use_cuda_graph=graphs, graph_after=1, max_shape_graphs=1000, **kw),
                        num_pages=num_pages)


TOL_SHARP = {"float32": 1e-4, "bfloat16": 0.12}


def check(models, name, dtype, steps, reqs, graphs=False, poison=True, tol=None, slots=4):
    name = pick(name, dtype)
    page = bz.PAGE[name[0]]
    cfg, w, _ = models[name]
    if tol is None:
        tol = bz.bound(dtype, cfg, w, reqs, TOL_SHARP[dtype] if "sharp" in name else None)
    runner = make_runner(models, name, dtype, max(ru.max_live_tokens(steps) // page, 1), graphs=graphs, slots=slots)
    got = ru.replay(runner, steps, poison=poison)
    worst = bz.compare(got, name, cfg, w, reqs, dtype, tol)
    assert runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in runner.manager.pools)
    return runner, got, worst


LENGTHS = {"A": [1, 2, 15, 16, 17, 47, 130], "B": [1, 7, 8, 9, 64, 120], "C": [3, 31, 32, 33, 129, 300], "D": [1, 16, 65, 140, 400]}


def requests_for(models, name):
    cfg = models[name][0]
    return {f"{name}{n}": bz.tokens(cfg, n, salt=len(name)) for n in LENGTHS[name[0]]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Asharp", "Csharp"])
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions"])
def test_each_request_alone(models, name, dtype, cut):
    """Whole prompts (lengths at and beside page borders and windows), prompt then token-by-token decoding, and portions
    of 1 to 31 tokens, each request by itself."""
    reqs = requests_for(models, name)
    check(models, name, dtype, getattr(ru, cut)(reqs), reqs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "Csharp"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_with_reused_pages_and_slots(models, name, dtype, seed):
    """Up to four live requests of unequal length, portions beside single tokens; nine requests through four state
    slots and fewer pages than they need together; what a freed page or slot held is overwritten with NaN."""
    cfg = models[name][0]
    reqs = {f"m{i}": bz.tokens(cfg, n, salt=seed + 3) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
    steps = ru.mixed(reqs, seed=seed)
    assert ru.max_live_tokens(steps) < sum(ru.ceil64(len(v)) for v in reqs.values())
    check(models, name, dtype, steps, reqs, slots=4)
    assert max(len(s["entries"]) for s in steps) >= 3


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("cut", ["tail_decoded", "portions", "mixed_decodes_first"])
def test_every_cutting_through_recorded_graphs(models, name, cut):
    """bfloat16 with recordings on: the trace runs twice through one runner; the second pass replays the CUDA graphs
    the first recorded, with other pages and slots under the same requests."""
    name = pick(name, "bfloat16")
    cfg, w, _ = models[name]
    if cut.startswith("mixed"):
        reqs = {f"m{i}": bz.tokens(cfg, n, salt=5) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
        steps = ru.mixed(reqs, seed=4, decodes_first=True)
    else:
        reqs = requests_for(models, name)
        steps = getattr(ru, cut)(reqs)
    page = bz.PAGE[name[0]]
    runner = make_runner(models, name, "bfloat16", max(ru.max_live_tokens(steps) // page, 1), graphs=True)
    assert runner._can_record
    tol = bz.bound("bfloat16", cfg, w, reqs)
    first = ru.replay(runner, steps, poison=True)
    bz.compare(first, name, cfg, w, reqs, "bfloat16", tol)
    recorded, replays = len(runner._graphs), runner.graph_replays
    assert recorded > 0
    second = ru.replay(runner, steps, poison=True)
    bz.compare(second, name, cfg, w, reqs, "bfloat16", tol)
    assert len(runner._graphs) == recorded and runner.graph_replays - replays == sum(1 for s in steps if s["entries"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_cutting_does_not_change_float32_results_at_all(models, name, dtype):
    """In 32-bit every sum's order is fixed by the model's sizes alone, so whole prompts, portions, single tokens and
    mixed batches agree to the last bit; in bfloat16 within rounding."""
    name = pick(name, dtype)
    reqs = requests_for(models, name)
    runs = []
    for steps in (ru.whole(reqs), ru.portions(reqs), ru.mixed(reqs, seed=3), ru.tail_decoded(reqs, tail=40)):
        runner = make_runner(models, name, dtype, 200)
        runs.append(ru.replay(runner, steps))
    common = set(runs[0]) & set(runs[1]) & set(runs[2])
    assert len(common) > 50
    for key in common:
        for other in runs[1:]:
            if key not in other:
                continue
            if dtype == "float32":
                assert torch.equal(runs[0][key], other[key]), key
            else:
                assert (runs[0][key] - other[key]).abs().max() <= 2 * bz.TOL[dtype] * runs[0][key].abs().max(), key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp", "D"])
def test_long_decoding_past_windows_with_old_state(models, name, dtype):
    """A short prompt, then hundreds of tokens decoded one by one: every window passes over decoded tokens (pages are
    given back as it does), and the slow decays still carry what entered the state at the start."""
    cfg = models[name][0]
    ids = bz.tokens(cfg, 390, salt=9)
    steps = ru.tail_decoded({"long": ids}, tail=387)
    _, got, _ = check(models, name, dtype, steps, {"long": ids})
    assert len(got) == 388


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Asharp", "Csharp"])
def test_the_windows_edges_really_matter(models, name, dtype):
    """The sharpened model must be one in which single keys matter: replacing the token that stands just inside the
    first layer's window of the last query changes the last logits by far more than the 32-bit tolerance.  Then the
    engine, the prompt in portions that end at, before and behind page borders, against the plain implementation."""
    mname = pick(name, dtype)
    cfg, w, _ = models[mname]
    window = cfg["layers"][0]["mixer"]["left"]["mask"]["size"]
    ids = bz.tokens(cfg, 200, salt=21)
    other = list(ids)
    other[199 - (window - 1)] = (ids[199 - (window - 1)] + 1) % cfg["vocab"]
    a, b = bz.plain_logits(mname, cfg, w, ids), bz.plain_logits(mname, cfg, w, other)
    assert (a[-1] - b[-1]).abs().max() > 20 * TOL_SHARP["float32"] * a.abs().max()
    page = bz.PAGE[name[0]]
    steps = ru.portions({"edge": ids}, sizes=(page - 1, 2, page, page + 1, 2 * page - 2, 3, 5 * page, 1, 1, 2))
    check(models, name, dtype, steps, {"edge": ids})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0 to 5: a single key, fewer tokens than a window holds, a page with one token, an empty state."""
    cfg = models[name][0]
    for n in (1, 2, 3, 6):
        ids = bz.tokens(cfg, n, salt=n)
        for steps in (ru.whole({"f": ids}), ru.tail_decoded({"f": ids}, tail=n - 1) if n > 1 else ru.whole({"f": ids})):
            check(models, name, dtype, steps, {"f": ids})


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_against_each_alone(models, dtype):
    """Five unequal prompts in one step, then their next tokens in one step: every row equals the request run alone."""
    name = "C"
    cfg = models[name][0]
    reqs = {f"b{n}": bz.tokens(cfg, n, salt=31) for n in (2, 40, 17, 128, 65)}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": ids[:-1], "want": [len(ids) - 2]} for r, ids in reqs.items()], "end": []},
             {"step": 1, "entries": [{"id": r, "tokens": ids[-1:], "want": [0]} for r, ids in reqs.items()], "end": list(reqs)}]
    _, together, _ = check(models, name, dtype, steps, reqs, slots=8)
    for r, ids in reqs.items():
        _, alone, _ = check(models, name, dtype, ru.whole({r: ids}), {r: ids})
        for p in (len(ids) - 2, len(ids) - 1):
            if dtype == "float32":
                assert torch.equal(together[(r, p)], alone[(r, p)]), (r, p)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Every size drawn at random: the 32-bit engine must agree with the plain implementation to 32-bit rounding under
    every cutting; the bfloat16 engine (with routing that rounding cannot turn) within its bound."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    cfg = bz.random_config(seed)
    reqs = {f"q{i}": bz.tokens(cfg, n, salt=seed) for i, n in enumerate((1, 23, 97, 200, 64))}
    for dtype in DTYPES:
        w = bz.make_weights(cfg, 300 + seed, decisive=dtype == "bfloat16")
        folder = bz.write_model(tmp_path / f"model_{dtype}", cfg, w)
        for cut in ("whole", "portions", "mixed", "tail_decoded"):
            steps = getattr(ru, cut)(reqs)
            pages = max(ru.max_live_tokens(steps) // 16, 1)
            runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_blocks=pages, max_num_seqs=4,
                                                        use_cuda_graph=(cut == "mixed"), graph_after=1), num_pages=pages)
            got = ru.replay(runner, steps, poison=True)
            bz.compare(got, ("drawn", seed, dtype), cfg, w, reqs, dtype, tol=3e-5 if dtype == "float32" else bz.bound(dtype, cfg, w, reqs, 5e-2))


# ---- through the entry point -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, slack):
    """Engine.generate with the scheduler's own batching: prompts longer than a step's budget (so they are read in
    portions beside decoding requests), more requests than state slots.  Every generated token must be the plain
    implementation's choice for the same prefix, or lose to it by a near-tie."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    name = pick(name, dtype)
    cfg, w, folder = models[name]
    eng = Engine(folder, options=EngineOptions(dtype=dtype, block_size=bz.PAGE[name[0]], max_blocks=64, max_tokens_per_step=48, max_num_seqs=3))
    prompts = [bz.tokens(cfg, n, salt=41) for n in (5, 70, 33, 1, 100)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert all(len(o) == 6 for o in outs)
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for k, tok in enumerate(out):
            row = bz.plain_logits(name, cfg, w, ids)[-1]
            assert row.max() - row[tok] <= slack * row.abs().max().clamp(min=1.0), f"token {k}: chose {tok}, plain chooses {int(row.argmax())}"
            ids.append(tok)
    assert eng.runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in eng.runner.manager.pools)


def test_generation_under_page_pressure_recomputes_the_state(models):
    """Fewer pages than the requests need together: a request is preempted, gives its pages and its slot back and is
    recomputed later from its prompt and what it had generated; the output is the same as with pages to spare."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models["D"]                # its first layer's window is longer than the sequences: pages are kept
    prompts = [bz.tokens(cfg, n, salt=51) for n in (60, 50, 40, 30)]
    params = SamplingParams(max_new_tokens=40, ignore_eos=True)
    roomy = Engine(folder, options=EngineOptions(dtype="float32", block_size=16, max_blocks=64, max_tokens_per_step=64, max_num_seqs=4))
    want = roomy.generate(prompts, params)
    tight = Engine(folder, options=EngineOptions(dtype="float32", block_size=16, max_blocks=16, max_tokens_per_step=64, max_num_seqs=4))
    got = tight.generate(prompts, params)
    assert got == want
    assert tight.stats()["preemptions"] > 0 and roomy.stats()["preemptions"] == 0


# ---- the programs ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_trace_run_program(models, tmp_path, dtype, graphs):
    """bin/trace_run as a user runs it on a Bonolorn folder: the model is chosen by config.json, steps come on standard
    input, <step>.f32 files go out; six requests through its four state slots."""
    import json
    import subprocess
    import sys

    import numpy as np

    from conftest import ROOT
    name = pick("A", dtype)
    cfg, w, folder = models[name]
    reqs = {f"t{i}": bz.tokens(cfg, n, salt=61) for i, n in enumerate((70, 33, 90, 5, 64, 41))}
    steps = ru.mixed(reqs, seed=5, max_live=4)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(ru.max_live_tokens(steps))] + (["--cuda-graph"] if graphs else []),
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, held = {}, {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        assert f.exists() == (wanted > 0)
        rows = np.fromfile(f, dtype="<f4").reshape(wanted, cfg["vocab"]) if wanted else None
        r = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for k in e["want"]:
                got[(e["id"], start + k)] = torch.from_numpy(rows[r].astype(np.float64)); r += 1
            held[e["id"]] = start + len(e["tokens"])
    bz.compare(got, name, cfg, w, reqs, dtype)


def test_chat_program_and_random_model_program(tmp_path):
    """bin/lucciola_random_model writes a Bonolorn folder from a config.json; bin/lucciola_chat generates from it, and
    its greedy tokens are the plain implementation's."""
    import json
    import subprocess
    import sys

    from conftest import ROOT
    from lucciola_b200.weights.safetensors_io import SafetensorsFile
    cfg = bz.CONFIGS["B"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_random_model"), "--config", str(tmp_path / "config.json"), "--seed", "3",
                        "--out", str(folder), "--std", "0.3", "--norm-std", "0.1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    prompt = bz.tokens(cfg, 19, salt=71)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_chat"), "--model", str(folder), "--dtype", "float32", "--max-blocks", "32",
                        "--block-size", "8", "--max-new-tokens", "5", "--ignore-eos", "--prompt-ids", " ".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()[-5:]]
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.get(n).clone() for n in f.names()}
    ids = list(prompt)
    for tok in out:
        row = plain.PlainBonolorn(cfg, w).forward(ids)[-1]
        assert row.max() - row[tok] <= 1e-4 * row.abs().max(), (tok, int(row.argmax()))
        ids.append(tok)
