"""Riruzen in the engine against the plain implementation: every mechanism alone, then the whole model under every
way of cutting the work, with pages and state slots that are freed and used again, and generation through the entry
point (GPU)."""
from types import SimpleNamespace

import pytest
import torch

import plain_riruzen as plain
import replay_util as ru
import riruzen_util as rz

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
                           positions=i32(pos))


# ---- each mechanism alone --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("hidden,groups", [(72, 3), (40, 1), (256, 2), (48, 4), (4096, 4), (1536, 1), (640, 40), (96, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_norm_with_two_deltas(hidden, groups, dtype):
    from lucciola_b200 import ops
    T = 5
    r = torch.randn(T, hidden, device=DEV) * 3
    a, b = (torch.randn(T, hidden, device=DEV).to(dtype) for _ in range(2))
    w = 1 + 0.3 * torch.randn(hidden, device=DEV)
    want_sum = r.double() + a.double() + b.double()
    want = plain.group_rms_norm(want_sum.cpu(), w.double().cpu(), groups, 1e-5)
    out, res = torch.empty(T, hidden, dtype=dtype, device=DEV), r.clone()
    ops.add_group_rmsnorm(out, res, (a, b), w, groups, 1e-5, stream())
    assert torch.allclose(res.double(), want_sum.float().double(), atol=1e-6)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    # on chosen rows, with one delta, the residual stays as it is
    rows = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    out2, res2 = torch.empty(3, hidden, dtype=dtype, device=DEV), r.clone()
    ops.add_group_rmsnorm(out2, res2, (a,), w, groups, 1e-5, stream(), rows=rows)
    want2 = plain.group_rms_norm((r.double() + a.double()).cpu()[[4, 0, 2]], w.double().cpu(), groups, 1e-5)
    assert torch.equal(res2, r) and (out2.double().cpu() - want2).abs().max() <= tol * want2.abs().max()


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_causal_taps_over_portions_of_several_sequences(taps, dtype):
    """Three sequences move on side by side in portions of 1, 2, 3, ... tokens (shorter and longer than the taps
    reach); each must equal the convolution of its whole."""
    from lucciola_b200 import ops
    W, slots = 70, [2, 0, 3]
    w = torch.randn(W, taps, device=DEV)
    full = [torch.randn(n, W, device=DEV).to(dtype) for n in (11, 17, 6)]
    want = [plain.causal_taps(h.double().cpu(), w.double().cpu()) + h.double().cpu() for h in full]
    state = torch.zeros(5, max(taps - 1, 0), W, dtype=dtype, device=DEV) if taps > 1 else None
    at, got = [0, 0, 0], [[], [], []]
    sizes = [1, 2, 1, 3, 4, 1, 7, 2, 30]
    k = 0
    while any(a < len(f) for a, f in zip(at, full)):
        live = [i for i in range(3) if at[i] < len(full[i])]
        lens = [min(sizes[(k + i) % len(sizes)], len(full[i]) - at[i]) for i in live]
        k += 1
        h = torch.cat([full[i][at[i]:at[i] + n] for i, n in zip(live, lens)])
        step = batch_of(lens, [slots[i] for i in live])
        out = torch.empty_like(h)
        ops.causal_taps(out, h, w.t().contiguous(), state, step, stream())
        if taps > 1:
            ops.causal_taps_state(state, h, taps, step, stream())
        o = 0
        for i, n in zip(live, lens):
            got[i].append(out[o:o + n]); o += n; at[i] += n
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    for i in range(3):
        g = torch.cat(got[i]).double().cpu()
        assert (g - want[i]).abs().max() <= tol * want[i].abs().max(), i
    if taps > 1:
        assert torch.equal(state[1], torch.zeros_like(state[1])) and torch.equal(state[2].cpu(), full[0][-(taps - 1):].cpu())


@pytest.mark.parametrize("heads,dim,vdim", [(2, 20, 40), (1, 40, 40), (3, 36, 12), (2, 128, 64), (4, 64, 128), (6, 8, 8), (1, 200, 33), (1, 256, 5), (1, 300, 40), (1, 1000, 8)])
def test_gated_recurrence_alone(heads, dim, vdim):
    """Two sequences in unequal portions, against the plain recurrence with the output map left out (identity)."""
    from lucciola_b200 import ops
    n = heads * dim
    W = 2 * n + heads * vdim
    lens_total, slots = (37, 5), [1, 3]
    pre = [torch.randn(t, W, device=DEV) for t in lens_total]
    bias, lower = torch.randn(n, device=DEV), torch.rand(n, device=DEV)
    norm_w = 1 + 0.2 * torch.randn(vdim, device=DEV)
    state = torch.zeros(5, heads, dim, vdim, device=DEV)
    state[2] = float("nan")                                                   # a row of another request
    got = [[], []]
    at = [0, 0]
    for sizes in ([1, 2], [17, 1], [3, 1], [16, 1], [0, 0]):
        live = [i for i in range(2) if at[i] < lens_total[i] and sizes[i]]
        if not live:
            continue
        lens = [min(sizes[i], lens_total[i] - at[i]) for i in live]
        x = torch.cat([pre[i][at[i]:at[i] + k] for i, k in zip(live, lens)])
        out = torch.empty(x.shape[0], heads * vdim, device=DEV)
        # steps of a few tokens a sequence, when the caller says so, run in a kernel of their own
        ops.gated_recurrence(x, 0, n, 2 * n, bias, lower, state, out, batch_of(lens, [slots[i] for i in live]), heads, dim, vdim, stream(),
                             max_tokens_a_seq=max(lens) if max(lens) <= 3 else 0)
        o = 0
        for i, k in zip(live, lens):
            got[i].append(out[o:o + k]); o += k; at[i] += k
    assert at == list(lens_total)
    # the plain function takes the projections' weights: identities make its input the pre-activations themselves
    eye = torch.eye(W, dtype=torch.float64)
    w = {"q": eye[:n], "f": eye[n:2 * n], "v": eye[2 * n:], "f.b": bias.double().cpu(), "lower": lower.double().cpu(),
         "norm": norm_w.double().cpu(), "o": torch.eye(heads * vdim, dtype=torch.float64)}
    for i in range(2):
        want, S = plain.hgrn2(pre[i].double().cpu(), w, heads, dim, vdim, 1e-6)
        o = torch.cat(got[i]).double().cpu().view(-1, heads, vdim)
        o = (o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.double().cpu()).reshape(-1, heads * vdim)
        assert (o - want).abs().max() <= 2e-5 * want.abs().max(), i
        assert (state[slots[i]].double().cpu() - S).abs().max() <= 1e-5 * S.abs().max()
    assert torch.isnan(state[2]).all() and torch.equal(state[0], torch.zeros_like(state[0]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_norm_writes_the_right_places(dtype):
    from lucciola_b200 import ops
    q_rank, kv_rank, page = 24, 40, 4
    lens, starts = [3, 1, 6], [0, 9, 2]
    step = batch_of(lens, [0, 1, 2], starts)
    T = sum(lens)
    pre = torch.randn(T, q_rank + kv_rank + 7, device=DEV) * 2
    qw, kw = 1 + 0.2 * torch.randn(q_rank, device=DEV), 1 + 0.2 * torch.randn(kv_rank, device=DEV)
    table = torch.tensor([[5, -1, -1], [0, 1, 7], [2, 3, -1]], dtype=torch.int32, device=DEV)
    pages = torch.full((8, 1, page, kv_rank), 99.0, dtype=dtype, device=DEV)
    cq = torch.empty(T, q_rank, dtype=dtype, device=DEV)
    ops.latent_norm(pre, 0, q_rank, q_rank, kv_rank, qw, kw, cq, pages, step, table, page, 1e-6, stream())
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    want_q = plain.rms_norm(pre[:, :q_rank].double().cpu(), qw.double().cpu(), 1e-6)
    want_c = plain.rms_norm(pre[:, q_rank:q_rank + kv_rank].double().cpu(), kw.double().cpu(), 1e-6)
    assert (cq.double().cpu() - want_q).abs().max() <= tol * want_q.abs().max()
    written = set()
    for t in range(T):
        s, p = int(step.token_seq[t]), int(step.positions[t])
        pg = int(table[s, p // page])
        written.add((pg, p % page))
        assert (pages[pg, 0, p % page].double().cpu() - want_c[t]).abs().max() <= tol * want_c.abs().max(), t
    for pg in range(8):
        for sl in range(page):
            if (pg, sl) not in written:
                assert (pages[pg, 0, sl] == 99.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,K,N", [(70, 3, 28, 20), (130, 5, 64, 48), (1, 2, 128, 128), (515, 2, 72, 130), (9, 1, 8, 3)])
def test_products_a_head_with_and_without_gate(dtype, T, H, K, N):
    """Sizes the tensor-core kernel takes in bfloat16 (K a multiple of 8) and sizes that go to the plain kernel."""
    from lucciola_b200 import ops
    x, w = torch.randn(T, H, K, device=DEV).to(dtype), torch.randn(H, N, K, device=DEV).to(dtype)
    gate = torch.randn(T, H * N + 5, device=DEV)[:, 5:]
    y, z = torch.empty(T, H, N, dtype=dtype, device=DEV), torch.empty(T, H, N, dtype=dtype, device=DEV)
    ops.gemm_heads(y, x, w, stream())
    ops.gemm_heads(z, x, w, stream(), gate=gate)
    want = torch.einsum("thk,hnk->thn", x.double(), w.double())
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert (y.double() - want).abs().max() <= tol * want.abs().max()
    want = want * torch.sigmoid(gate.double()).view(T, H, N)
    assert (z.double() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_relu_gate_and_embedding_with_positions(dtype):
    from lucciola_b200 import ops
    T, inter, K = 9, 128, 64
    gu = torch.randn(T, 2 * inter, device=DEV).to(dtype)
    out = torch.empty(T, inter, dtype=dtype, device=DEV)
    ops.swiglu(out, gu[:, :inter], gu[:, inter:], stream(), act="relu")
    want = torch.relu(gu[:, :inter].double()) * gu[:, inter:].double()
    assert (out.double() - want).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()
    if dtype == torch.bfloat16:                        # the same inside the tensor-core product's epilogue, few tokens and many
        for M in (3, 200):
            x = torch.randn(M, K, device=DEV).to(dtype)
            gate, up = (torch.randn(inter, K, device=DEV).to(dtype) * 0.2 for _ in range(2))
            act = torch.empty(M, inter, dtype=dtype, device=DEV)
            ops.gemm_tcgen05(act, x, ops.interleave_gate_up(gate, up), stream(), swiglu=True, act="relu")
            want = torch.relu(x.double() @ gate.double().T) * (x.double() @ up.double().T)
            assert (act.double() - want).abs().max() <= 1e-2 * want.abs().max(), M
    table, pos = torch.randn(30, 48, device=DEV).to(dtype), torch.randn(50, 48, device=DEV).to(dtype)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32, device=DEV)
    at = torch.tensor([0, 49, 7, 8], dtype=torch.int32, device=DEV)
    x = torch.empty(4, 48, device=DEV)
    ops.embedding(x, ids, table, stream(), pos_table=pos, positions=at)
    assert torch.equal(x, table[ids.long()].float() + pos[at.long()].float())
    ops.scale_(x, 0.37, stream())
    assert torch.equal(x, (table[ids.long()].float() + pos[at.long()].float()) * 0.37)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,page", [(3, 28, 8), (4, 64, 16), (8, 128, 16), (2, 40, 4), (1, 200, 16), (32, 128, 16), (24, 64, 8),
                                             (20, 32, 16), (17, 64, 16), (64, 128, 32)])
def test_a_query_finds_its_one_key_anywhere(dtype, heads, rank, page):
    """Attention over pages that hold one latent a token as key and value: every head of every query is made to
    point at one key of its own sequence (the first, the last it may see, keys at and beside page borders, keys
    hundreds of tokens back), with a score so far above the others that the result must be that key's latent itself.
    Three sequences of unequal length in one batch: a prompt's portion behind a cached part, a whole prompt, one
    decoded token; pages in scrambled order, every other page filled with NaN.  More than 16 heads are cut into groups
    that each read the one cached head (as the latent attention part asks for them)."""
    from lucciola_b200 import ops
    from lucciola_b200.parts import BatchShape, LatentAttention, PlanView, Runtime
    starts, lens = [300, 0, 517], [77, 130, 1]
    total = [s + n for s, n in zip(starts, lens)]
    max_pages = max(-(-t // page) for t in total)
    perm = torch.randperm(3 * max_pages + 5).tolist()
    table = torch.full((3, max_pages), -1, dtype=torch.int32)
    pool = torch.full((3 * max_pages + 5, 1, page, rank), float("nan"))
    lat = [torch.nn.functional.normalize(torch.randn(t, rank), dim=-1).mul(rank ** 0.5).to(dtype).float() for t in total]   # equal lengths
    for s in range(3):
        for i in range(-(-total[s] // page)):
            table[s, i] = perm.pop()
            chunk = lat[s][i * page:(i + 1) * page]
            pool[table[s, i], 0, :chunk.shape[0]] = chunk
    step = batch_of(lens, [0, 1, 2], starts)
    step.block_tables = [table.to(DEV)]
    step.q_lens, step.start_positions, step.max_q_len, step.max_context_len, step.span_hint = lens, starts, max(lens), max(total), 0
    T = sum(lens)
    q = torch.zeros(T, heads, rank)
    want = torch.zeros(T, heads, rank)
    t = 0
    for s in range(3):
        for j in range(lens[s]):
            p = starts[s] + j
            picks = [0, p, max(p - 1, 0), (p // page) * page, max((p // page) * page - 1, 0), p // 2, min(page, p), min(page - 1, p), p // 3]
            for h in range(heads):
                key = picks[(t + h) % len(picks)]
                c = lat[s][key]
                q[t, h] = c * (160.0 / c.pow(2).sum())           # its own score 160, another key's 160 x the cosine between the two
                want[t, h] = c
            t += 1
    part = LatentAttention(Runtime(DEV, dtype), "x", 8, heads, 8, 8, 8, rank, 1.0, 1e-6)
    assert heads // part.share <= 16 and heads % part.share == 0
    plan = part.plan(BatchShape(lens, starts, max(lens), max(total), max(total)))
    view = PlanView({k: torch.tensor(v, device=DEV) for k, v in plan.arrays.items()}, plan.host)
    q, pool = q.to(dtype).to(DEV), pool.to(dtype).to(DEV)
    out = torch.empty_like(q)
    ops.attention(q, out, pool, pool, step, 0, heads, 1, rank, page, 0, 1.0, stream(), plan=view if dtype == torch.bfloat16 else None,
                  kv_share=part.share)
    if heads == 32:                                    # single tokens alone: the decode kernel, two groups of 16 heads on the one cached head
        dec = batch_of([1, 1, 1], [0, 1, 2], [t - 1 for t in total])
        dec.block_tables, dec.q_lens, dec.start_positions = step.block_tables, [1, 1, 1], [t - 1 for t in total]
        dec.max_q_len, dec.max_context_len, dec.span_hint = 1, max(total), 0
        rows = [lens[0] - 1, lens[0] + lens[1] - 1, T - 1]        # the last token of each sequence, as computed above
        plan1 = part.plan(BatchShape([1, 1, 1], dec.start_positions, 1, max(total), max(total)))
        view1 = PlanView({k: torch.tensor(v, device=DEV) for k, v in plan1.arrays.items()}, plan1.host)
        q1, out1 = q[rows].contiguous(), torch.empty_like(q[rows])
        ops.attention(q1, out1, pool, pool, dec, 0, heads, 1, rank, page, 0, 1.0, stream(), plan=view1 if dtype == torch.bfloat16 else None,
                      kv_share=part.share)
        assert (out1.float().cpu() - want[rows]).abs().max().item() <= (2e-2 if dtype == torch.bfloat16 else 1e-4) * want.abs().max().item()
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= (2e-2 if dtype == torch.bfloat16 else 1e-4) * want.abs().max().item(), err


# ---- the whole model -------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, weights, folder); beside the four configurations: P with attention that picks out single keys
    anywhere in the sequence ("Psharp"), and P and S with recurrences that forget slowly ("Pkeep", "Skeep")."""
    out = {}
    for name, cfg in rz.CONFIGS.items():
        w = rz.make_weights(cfg, 100 + len(out))
        out[name] = (cfg, w, rz.write_model(tmp_path_factory.mktemp(f"riruzen_{name}"), cfg, w))
    for name, base, kw in (("Psharp", "P", dict(sharp=6.0)), ("Pkeep", "P", dict(keep=0.97)), ("Skeep", "S", dict(keep=0.98)),
                           ("Rsharp", "R", dict(sharp=5.0, keep=0.95))):
        cfg = rz.CONFIGS[base]
        w = rz.make_weights(cfg, 200 + len(out), **kw)
        out[name] = (cfg, w, rz.write_model(tmp_path_factory.mktemp(f"riruzen_{name}"), cfg, w))
    return out


def make_runner(models, name, dtype, num_pages, graphs=False, slots=4, **kw):
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    page = rz.PAGE[name[0]]
    return build_runner(models[name][2], EngineOptions(dtype=dtype, block_size=page, max_blocks=num_pages, max_num_seqs=slots,
                                                       use_cuda_graph=graphs, graph_after=1, max_shape_graphs=1000, **kw),
                        num_pages=num_pages)


# Attention that is sharpened until single keys carry a query's weight multiplies what the rounding of queries and
# latents does to the scores: such models are compared with a wider bound.  In 32-bit the change that lost far keys
# make exceeds it a thousand times (test_attention_weights_really_sit_on_far_keys); in bfloat16 rounding and a lost key
# are of one size in such a model, and the sharp test of far keys is test_a_query_finds_its_one_key_anywhere.
TOL_SHARP = {"float32": 1e-4, "bfloat16": 0.12}


# A recurrence that forgets slowly carries the 32-bit rounding of hundreds of updates in its state.
TOL_KEEP = {"float32": 5e-5, "bfloat16": rz.TOL["bfloat16"]}


def check(models, name, dtype, steps, reqs, graphs=False, poison=True, tol=None, slots=4):
    page = rz.PAGE[name[0]]
    if tol is None and name.endswith("sharp"):
        tol = TOL_SHARP[dtype]
    if tol is None and name.endswith("keep"):
        tol = TOL_KEEP[dtype]
    runner = make_runner(models, name, dtype, max(ru.max_live_tokens(steps) // page, 1), graphs=graphs, slots=slots)
    got = ru.replay(runner, steps, poison=poison)
    cfg, w, _ = models[name]
    worst = rz.compare(got, name, cfg, w, reqs, dtype, tol)
    assert runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in runner.manager.pools)
    return runner, got, worst


LENGTHS = {"P": [1, 2, 15, 16, 17, 47, 130], "Q": [1, 7, 8, 9, 64, 120], "R": [3, 31, 32, 33, 129, 300], "S": [1, 4, 5, 6, 77, 200],
           "T": [1, 2, 16, 63, 65, 140]}


def requests_for(models, name):
    cfg = models[name][0]
    return {f"{name}{n}": rz.tokens(cfg, n, salt=len(name)) for n in LENGTHS[name[0]]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "T", "Psharp", "Skeep"])
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions"])
def test_each_request_alone(models, name, dtype, cut):
    """Whole prompts (lengths at and beside page borders), prompt then token-by-token decoding, and portions of
    1 to 31 tokens, each request by itself."""
    reqs = requests_for(models, name)
    check(models, name, dtype, getattr(ru, cut)(reqs), reqs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "T", "Rsharp", "Pkeep"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_with_reused_pages_and_slots(models, name, dtype, seed):
    """Up to four live requests of unequal length, portions beside single tokens; nine requests through four state
    slots and fewer pages than they need together; what a freed page or slot held is overwritten with NaN."""
    cfg = models[name][0]
    reqs = {f"m{i}": rz.tokens(cfg, n, salt=seed + 3) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
    steps = ru.mixed(reqs, seed=seed)
    page = rz.PAGE[name[0]]
    assert ru.max_live_tokens(steps) < sum(ru.ceil64(len(v)) for v in reqs.values())
    check(models, name, dtype, steps, reqs, slots=4)
    assert max(len(s["entries"]) for s in steps) >= 3


@pytest.mark.parametrize("name", ["P", "Q", "R", "S", "T"])
@pytest.mark.parametrize("cut", ["tail_decoded", "portions", "mixed_decodes_first"])
def test_every_cutting_through_recorded_graphs(models, name, cut):
    """bfloat16 with recordings on: the trace runs twice through one runner; the second pass replays the CUDA graphs
    the first recorded, with other pages and slots under the same requests."""
    cfg, w, _ = models[name]
    if cut.startswith("mixed"):
        reqs = {f"m{i}": rz.tokens(cfg, n, salt=5) for i, n in enumerate((70, 9, 120, 33, 101, 2, 64, 47, 90))}
        steps = ru.mixed(reqs, seed=4, decodes_first=True)
    else:
        reqs = requests_for(models, name)
        steps = getattr(ru, cut)(reqs)
    page = rz.PAGE[name[0]]
    runner = make_runner(models, name, "bfloat16", max(ru.max_live_tokens(steps) // page, 1), graphs=True)
    assert runner._can_record
    first = ru.replay(runner, steps, poison=True)
    rz.compare(first, name, cfg, w, reqs, "bfloat16")
    recorded, replays = len(runner._graphs), runner.graph_replays
    assert recorded > 0
    second = ru.replay(runner, steps, poison=True)
    rz.compare(second, name, cfg, w, reqs, "bfloat16")
    assert len(runner._graphs) == recorded and runner.graph_replays - replays == sum(1 for s in steps if s["entries"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_cutting_does_not_change_float32_results_at_all(models, name, dtype):
    """In 32-bit every sum's order is fixed by the model's sizes alone, so whole prompts, portions, single tokens and
    mixed batches agree to the last bit; in bfloat16 within rounding."""
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
                assert (runs[0][key] - other[key]).abs().max() <= 2 * rz.TOL[dtype] * runs[0][key].abs().max(), key


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Psharp", "Skeep", "Rsharp"])
def test_long_decoding_with_far_keys_and_old_state(models, name, dtype):
    """A short prompt, then hundreds of tokens decoded one by one: attention that singles out keys anywhere in the
    past, and recurrent state that still carries what entered it long ago."""
    cfg = models[name][0]
    n = min(cfg["max_positions"], 390)
    ids = rz.tokens(cfg, n, salt=9)
    steps = ru.tail_decoded({"long": ids}, tail=n - 3)
    _, got, _ = check(models, name, dtype, steps, {"long": ids})
    assert len(got) == n - 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Psharp", "Rsharp"])
def test_attention_weights_really_sit_on_far_keys(models, name, dtype):
    """The sharpened model must be one in which far keys matter: with the first 200 tokens of a sequence of 300 replaced
    (all of them a hundred tokens and more behind the last) the last logits change by a thousand times the tolerance
    of the 32-bit comparison.  Then the engine, prompt in portions that end
    at, before and behind page borders, against the plain implementation."""
    cfg, w, _ = models[name]
    ids = rz.tokens(cfg, 300, salt=21)
    other = rz.tokens(cfg, 200, salt=22) + ids[200:]
    a, b = rz.plain_logits(name, cfg, w, ids), rz.plain_logits(name, cfg, w, other)
    assert (a[-1] - b[-1]).abs().max() > 1000 * TOL_SHARP["float32"] * a.abs().max()
    page = rz.PAGE[name[0]]
    steps = ru.portions({"far": ids}, sizes=(page - 1, 2, page, page + 1, 2 * page - 2, 3, 5 * page, 1, 1, 2))
    check(models, name, dtype, steps, {"far": ids})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0 to 5: fewer inputs than the convolution has taps, a single key, a page with one token."""
    cfg = models[name][0]
    for n in (1, 2, 3, 6):
        ids = rz.tokens(cfg, n, salt=n)
        for steps in (ru.whole({"f": ids}), ru.tail_decoded({"f": ids}, tail=n - 1) if n > 1 else ru.whole({"f": ids})):
            check(models, name, dtype, steps, {"f": ids})


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_against_each_alone(models, dtype):
    """Five unequal prompts in one step, then their next tokens in one step: every row equals the request run alone."""
    name = "R"
    cfg, w, _ = models[name]
    reqs = {f"b{n}": rz.tokens(cfg, n, salt=31) for n in (2, 40, 17, 128, 65)}
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
    every cutting; the bfloat16 engine within a few times what rounding the sublayers' inputs alone does to that model."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    cfg = rz.random_config(seed)
    w = rz.make_weights(cfg, 300 + seed)
    folder = rz.write_model(tmp_path / "model", cfg, w)
    reqs = {f"q{i}": rz.tokens(cfg, n, salt=seed) for i, n in enumerate((1, 23, 97, 200, 64))}
    floor = max(rz.rounding_alone(cfg, w, ids) for ids in reqs.values())
    for dtype in DTYPES:
        for cut in ("whole", "portions", "mixed", "tail_decoded"):
            steps = getattr(ru, cut)(reqs)
            pages = max(ru.max_live_tokens(steps) // 16, 1)
            runner = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_blocks=pages, max_num_seqs=4,
                                                        use_cuda_graph=(cut == "mixed"), graph_after=1), num_pages=pages)
            got = ru.replay(runner, steps, poison=True)
            rz.compare(got, ("drawn", seed), cfg, w, reqs, dtype, tol=3e-5 if dtype == "float32" else max(rz.TOL[dtype], 4 * floor))


# ---- through the entry point -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("name", ["P", "R", "S"])
def test_greedy_generation_through_the_entry_point(models, name, dtype, slack):
    """Engine.generate with the scheduler's own batching: prompts longer than a step's budget (so they are read in
    portions beside decoding requests), more requests than state slots.  Every generated token must be the plain
    implementation's choice for the same prefix, or lose to it by a near-tie."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models[name]
    eng = Engine(folder, options=EngineOptions(dtype=dtype, block_size=rz.PAGE[name[0]], max_blocks=64, max_tokens_per_step=48, max_num_seqs=3))
    prompts = [rz.tokens(cfg, n, salt=41) for n in (5, 70, 33, 1, 100)]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert all(len(o) == 6 for o in outs)
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for k, tok in enumerate(out):
            row = rz.plain_logits(name, cfg, w, ids)[-1]
            assert row.max() - row[tok] <= slack * row.abs().max().clamp(min=1.0), f"token {k}: chose {tok}, plain chooses {int(row.argmax())}"
            ids.append(tok)
    assert eng.runner.manager.num_requests() == 0 and all(p.num_free == p.num_pages for p in eng.runner.manager.pools)


def test_generation_under_page_pressure_recomputes_the_state(models):
    """Fewer pages than the requests need together: a request is preempted, gives its pages and its slot back and is
    recomputed later from its prompt and what it had generated; the output is the same as with pages to spare."""
    from lucciola_b200 import Engine, EngineOptions, SamplingParams
    cfg, w, folder = models["P"]
    prompts = [rz.tokens(cfg, n, salt=51) for n in (60, 50, 40, 30)]
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
    """bin/trace_run as a user runs it on a Riruzen folder: the model is chosen by config.json, steps come on standard
    input, <step>.f32 files go out; six requests through its four state slots."""
    import json
    import subprocess
    import sys

    import numpy as np

    from conftest import ROOT
    name = "P"
    cfg, w, folder = models[name]
    reqs = {f"t{i}": rz.tokens(cfg, n, salt=61) for i, n in enumerate((70, 33, 90, 5, 64, 41))}
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
    rz.compare(got, name, cfg, w, reqs, dtype)


def test_chat_program_and_random_model_program(tmp_path):
    """bin/lucciola_random_model writes a Riruzen folder from a config.json; bin/lucciola_chat generates from it, and
    its greedy tokens are the plain implementation's."""
    import json
    import subprocess
    import sys

    from conftest import ROOT
    from lucciola_b200.weights.safetensors_io import SafetensorsFile
    cfg = rz.CONFIGS["Q"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    folder = tmp_path / "model"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_random_model"), "--config", str(tmp_path / "config.json"), "--seed", "3",
                        "--out", str(folder), "--std", "0.3", "--norm-std", "0.1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    prompt = rz.tokens(cfg, 19, salt=71)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "lucciola_chat"), "--model", str(folder), "--dtype", "float32", "--max-blocks", "32",
                        "--block-size", "8", "--max-new-tokens", "5", "--ignore-eos", "--prompt-ids", " ".join(map(str, prompt))],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()[-5:]]
    f = SafetensorsFile(folder / "model.safetensors")
    w = {n: f.get(n).clone() for n in f.names()}
    ids = list(prompt)
    for tok in out:
        row = plain.PlainRiruzen(cfg, w).forward(ids)[-1]
        assert row.max() - row[tok] <= 1e-4 * row.abs().max(), (tok, int(row.argmax()))
        ids.append(tok)
