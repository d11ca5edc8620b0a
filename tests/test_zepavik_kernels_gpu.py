"""The mechanisms of the Zepavik decoder one at a time, each kernel against the plain implementation's function
or a computation written out in double: the summed embedding and its per-sequence state, the finish of the
fused projection (biases, value norm, cache write), attention with a distance bias, a window and a gate in
the kernel with run-time head sizes and in the kernels built for one head size, and the projection that
stores an activation.  Where random numbers would hide a lost key, one key is made to dominate."""
import math

import numpy as np
import pytest
import torch

import plain_zepavik

pytestmark = pytest.mark.gpu


def kernels(dtype, head_dim=16):
    from stratakv_b200 import ops
    return ops.kernels_for(dtype, head_dim, verbose=False)


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ---- embedding -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_summed_embedding_and_the_token_it_remembers(dtype):
    vocab, hidden, buckets, mul_prev, mul_cur, positions = 50, 24, 7, 20000003, 10000019, 40
    g = torch.Generator().manual_seed(3)
    table = torch.randn(vocab, hidden, generator=g).to(dtype)
    pair = torch.randn(buckets + 1, hidden, generator=g).to(dtype)
    where = torch.randn(positions, hidden, generator=g).to(dtype)
    weights = {"embed": table.double(), "bigram": pair.double(), "pos": where.double()}
    config = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    ops = kernels(dtype)
    last_ids = torch.full((2 * 5,), 49, dtype=torch.int32, device="cuda")       # what earlier users of the slots left
    dev = lambda t: t.cuda()
    seq_a = [int(t) for t in torch.randint(0, vocab, (11,), generator=g)]
    seq_b = [int(t) for t in torch.randint(0, vocab, (6,), generator=g)]
    want_a = plain_zepavik.embed(config, weights, seq_a).numpy()
    want_b = plain_zepavik.embed(config, weights, seq_b).numpy()

    def step(parts):
        """parts: (slot, tokens, first position) per sequence -> rows of the stream"""
        ids = [t for _, tokens, _ in parts for t in tokens]
        pos = [first + i for _, tokens, first in parts for i in range(len(tokens))]
        seq = [s for s, (_, tokens, _) in enumerate(parts) for _ in tokens]
        cu = np.cumsum([0] + [len(tokens) for _, tokens, _ in parts]).tolist()
        out = torch.empty(len(ids), hidden, dtype=torch.float32, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.embed_sum(dev(table), i32(ids), out, i32(pos), i32(seq), i32(cu), i32([slot for slot, _, _ in parts]), flag,
                      pair_table=dev(pair), last_ids=last_ids, mul_prev=mul_prev, mul_cur=mul_cur, position_table=dev(where))
        assert int(flag) == 0
        return out.cpu().numpy()

    # a prompt each (slots 3 and 1), then portions and single tokens; the first token reads the table's last row
    got = step([(3, seq_a[:4], 0), (1, seq_b[:1], 0)])
    np.testing.assert_allclose(got, np.concatenate([want_a[:4], want_b[:1]]), rtol=1e-6, atol=1e-6)
    got = step([(1, seq_b[1:2], 1), (3, seq_a[4:5], 4)])
    np.testing.assert_allclose(got, np.concatenate([want_b[1:2], want_a[4:5]]), rtol=1e-6, atol=1e-6)
    got = step([(3, seq_a[5:9], 5)])
    np.testing.assert_allclose(got, want_a[5:9], rtol=1e-6, atol=1e-6)
    # the same step twice (an eager run before a graph's capture, then the graph) reads the same previous token
    for _ in range(2):
        got = step([(3, seq_a[9:10], 9), (1, seq_b[2:3], 2)])
        np.testing.assert_allclose(got, np.concatenate([want_a[9:10], want_b[2:3]]), rtol=1e-6, atol=1e-6)
    got = step([(3, seq_a[10:11], 10)])
    np.testing.assert_allclose(got, want_a[10:11], rtol=1e-6, atol=1e-6)
    # a new sequence in a used slot starts from the last row whatever the slot remembers
    got = step([(3, seq_b[:2], 0)])
    np.testing.assert_allclose(got, want_b[:2], rtol=1e-6, atol=1e-6)


def test_embedding_flags_a_position_beyond_its_table():
    ops = kernels(torch.float32)
    table = torch.randn(10, 8, device="cuda")
    where = torch.randn(4, 8, device="cuda")
    out = torch.empty(1, 8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_sum(table, i32([2]), out, i32([4]), i32([0]), i32([0, 1]), i32([0]), flag, position_table=where)
    assert int(flag) == 8


# ---- finish of the fused projection -----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 16, 16), (6, 2, 20, 12), (3, 1, 24, 40), (1, 1, 8, 8)])
def test_qkv_finish_adds_biases_norms_values_and_fills_the_cache(dtype, heads, kv_heads, dim, vdim):
    ops = kernels(dtype)
    n, block_size, blocks, eps = 9, 16, 5, 1e-3
    width = (heads + kv_heads) * dim + kv_heads * vdim
    stride = -(-(width + heads) // 8) * 8
    g = torch.Generator().manual_seed(heads * 100 + dim)
    rows = torch.randn(n, stride, generator=g)
    biases = [torch.randn(heads * dim, generator=g), torch.randn(kv_heads * dim, generator=g), torch.randn(kv_heads * vdim, generator=g)]
    positions = [14, 15, 16, 17, 0, 1, 2, 31, 32]                # two sequences; pages 3, 1 and 0, 4, 2
    token_seq = [0, 0, 0, 0, 1, 1, 1, 1, 1]
    table = i32([[3, 1, 0], [0, 4, 2]])
    q = torch.empty(n, heads * dim, dtype=dtype, device="cuda")
    k_cache = torch.zeros(blocks, kv_heads, block_size, dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros(blocks, kv_heads, block_size, vdim, dtype=dtype, device="cuda")
    ops.qkv_finish(rows.cuda(), q, k_cache, v_cache, i32(positions), i32(token_seq), table, heads, kv_heads, dim, vdim,
                   block_size, *[b.cuda() for b in biases], value_norm_eps=eps)
    tol = dict(rtol=1e-6, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    rows64 = rows.double()
    want_q = rows64[:, :heads * dim] + biases[0].double()
    np.testing.assert_allclose(q.double().cpu().numpy(), want_q.numpy(), **tol)
    want_k = (rows64[:, heads * dim:(heads + kv_heads) * dim] + biases[1].double()).view(n, kv_heads, dim)
    want_v = (rows64[:, (heads + kv_heads) * dim:width] + biases[2].double()).view(n, kv_heads, vdim)
    want_v = plain_zepavik.rms_divide(want_v, eps)
    pages = table.cpu().tolist()
    written = torch.zeros(blocks, block_size, dtype=torch.bool)
    for t in range(n):
        page, row = pages[token_seq[t]][positions[t] // block_size], positions[t] % block_size
        written[page, row] = True
        np.testing.assert_allclose(k_cache[page, :, row].double().cpu().numpy(), want_k[t].numpy(), **tol)
        np.testing.assert_allclose(v_cache[page, :, row].double().cpu().numpy(), want_v[t].numpy(), **tol)
    assert float(k_cache.float().abs().sum(dim=(1, 3)).cpu()[~written].sum()) == 0.0      # nothing else was touched


# ---- attention ------------------------------------------------------------------------------------------
def plain_attention(q, k, v, scale, window, r1, r2, gate, kv_heads):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of ONE sequence (double) -> [T, H, dv]"""
    T, H, _ = q.shape
    seen = plain_zepavik.visible(T, window)
    penalty = plain_zepavik.distance_penalty(r1, r2, T) if r1 is not None else torch.zeros(H, T, T, dtype=torch.float64)
    out = []
    for head in range(H):
        kv = head // (H // kv_heads)
        score = (q[:, head] @ k[:, kv].T) * scale - penalty[head]
        weights = torch.softmax(score.masked_fill(~seen, -math.inf), dim=-1)
        o = weights @ v[:, kv]
        out.append(o * torch.sigmoid(gate[:, head:head + 1]) if gate is not None else o)
    return torch.stack(out, dim=1)


class Scene:
    """Sequences with keys and values already in a paged cache (pages handed out in a scrambled order), and the
    queries of each sequence's last `new` tokens."""

    def __init__(self, dtype, lengths, new, heads, kv_heads, dim, vdim, block_size, seed, loud=()):
        g = torch.Generator().manual_seed(seed)
        self.dtype, self.lengths, self.new = dtype, lengths, new
        self.heads, self.kv_heads, self.dim, self.vdim, self.block_size = heads, kv_heads, dim, vdim, block_size
        per_seq = [-(-length // block_size) for length in lengths]
        order = torch.randperm(sum(per_seq) + 2, generator=g).tolist()
        self.tables, at = [], 0
        for count in per_seq:
            self.tables.append(order[at:at + count])
            at += count
        width = max(per_seq)
        self.table = i32([row + [0] * (width - len(row)) for row in self.tables])
        blocks = sum(per_seq) + 2
        # stale rows everywhere: what a kernel must not read is large
        self.k_cache = torch.full((blocks, kv_heads, block_size, dim), 30.0, dtype=dtype, device="cuda")
        self.v_cache = torch.full((blocks, kv_heads, block_size, vdim), 1000.0, dtype=dtype, device="cuda")
        self.q, self.k, self.v = [], [], []
        for s, length in enumerate(lengths):
            q = torch.randn(length, heads, dim, generator=g).to(dtype)
            k = torch.randn(length, kv_heads, dim, generator=g).to(dtype)
            v = torch.randn(length, kv_heads, vdim, generator=g).to(dtype)
            for query, key in loud:                          # (query position from the end, key distance) made to dominate
                i = length - 1 - query
                j = i - key
                if 0 <= j <= i:
                    k[j] = (q[i, ::heads // kv_heads].float() * 3.0).to(dtype)
            self.q.append(q); self.k.append(k); self.v.append(v)
            for p in range(length):
                page, row = self.tables[s][p // block_size], p % block_size
                self.k_cache[page, :, row] = k[p].cuda()
                self.v_cache[page, :, row] = v[p].cuda()
        self.q_rows = torch.cat([q[length - n:] for q, length, n in zip(self.q, lengths, new)]).reshape(-1, heads * dim).cuda()
        self.positions = i32([p for length, n in zip(lengths, new) for p in range(length - n, length)])
        self.token_seq = i32([s for s, n in enumerate(new) for _ in range(n)])
        self.cu_q = i32(np.cumsum([0] + list(new)).tolist())
        self.ctx_after = i32(list(lengths))

    def plain(self, scale, window, r1, r2, gate):
        rows, at = [], 0
        for s, (length, n) in enumerate(zip(self.lengths, self.new)):
            whole_gate = None
            if gate is not None:
                whole_gate = torch.zeros(length, self.heads, dtype=torch.float64)
                whole_gate[length - n:] = gate[at:at + n].double().cpu()
            out = plain_attention(self.q[s].double(), self.k[s].double(), self.v[s].double(), scale, window,
                                  r1.double().cpu() if r1 is not None else None, r2.double().cpu() if r2 is not None else None,
                                  whole_gate, self.kv_heads)
            rows.append(out[length - n:].reshape(n, -1))
            at += n
        return torch.cat(rows).numpy()


SHAPES = [(4, 2, 16, 16), (6, 2, 20, 12), (3, 1, 24, 40), (2, 2, 64, 64), (8, 1, 32, 32)]
# (query from the end, distance of the key made loud): the query's own key, its neighbour, the window's last key inside
# and the first outside for windows of 24 and 100, a page border, a key far back
LOUD = [(0, 0), (1, 1), (2, 23), (3, 24), (4, 99), (5, 100), (6, 64), (7, 63), (8, 250)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 24, 100])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", SHAPES)
def test_attention_with_run_time_sizes(dtype, window, heads, kv_heads, dim, vdim):
    ops = kernels(dtype)
    scene = Scene(dtype, [300, 1, 70, 130], [40, 1, 70, 9], heads, kv_heads, dim, vdim, 64, seed=dim + window, loud=LOUD)
    g = torch.Generator().manual_seed(1)
    r1 = (torch.rand(heads, generator=g) + 0.1).cuda()
    r2 = (torch.rand(heads, generator=g) * 2 + 0.05).cuda()
    n = scene.q_rows.shape[0]
    stride = heads + 3
    gate = torch.randn(n, stride, generator=g).cuda()
    out_width = -(-heads * vdim // 8) * 8 + 8
    out = torch.full((n, out_width), 7.0, dtype=dtype, device="cuda")
    ops.attention_general(scene.q_rows, scene.k_cache, scene.v_cache, scene.table, scene.positions, scene.token_seq, out,
                          heads, kv_heads, dim, vdim, 64, 0.3, window, r1, r2, gate, stride)
    want = scene.plain(0.3, window, r1, r2, gate[:, :heads])
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(out[:, :heads * vdim].double().cpu().numpy(), want, **tol)
    assert float(out[:, heads * vdim:].float().abs().sum()) == 0.0          # the padding of a row is zeroed
    # without the bias and the gate the same kernel is plain windowed attention
    out2 = torch.empty((n, heads * vdim), dtype=dtype, device="cuda")
    ops.attention_general(scene.q_rows, scene.k_cache, scene.v_cache, scene.table, scene.positions, scene.token_seq, out2,
                          heads, kv_heads, dim, vdim, 64, 0.3, window)
    np.testing.assert_allclose(out2.double().cpu().numpy(), scene.plain(0.3, window, None, None, None), **tol)


def bias_table(r1, r2, reach):
    distance = torch.arange(reach, dtype=torch.float64)[None, :]
    natural = r1.double().cpu()[:, None] * torch.log1p(r2.double().cpu()[:, None] * distance)
    return (natural * math.log2(math.e)).float().cuda()          # the kernels take it in units of log2


@pytest.mark.parametrize("window", [0, 24, 100])
@pytest.mark.parametrize("heads,kv_heads,dim", [(4, 2, 16), (2, 2, 64), (8, 1, 32), (20, 1, 64), (2, 1, 128)])
def test_attention_kernels_of_one_head_size_take_the_bias_and_the_gate(window, heads, kv_heads, dim):
    """Prefill on tcgen05 (head sizes 64 and 128) and on mma.sync, and split decode, with the bias as a table."""
    dtype = torch.bfloat16
    ops = kernels(dtype, dim)
    g = torch.Generator().manual_seed(2)
    r1 = (torch.rand(heads, generator=g) + 0.1).cuda()
    r2 = (torch.rand(heads, generator=g) * 2 + 0.05).cuda()
    tol = dict(rtol=2e-2, atol=2e-2)
    # prompts and portions of prompts
    scene = Scene(dtype, [300, 33, 70, 200], [300, 33, 40, 129], heads, kv_heads, dim, dim, 64, seed=dim + window, loud=LOUD)
    n = scene.q_rows.shape[0]
    gate = torch.randn(n, heads + 1, generator=g).cuda()
    table = bias_table(r1, r2, window or 300)
    want = scene.plain(0.3, window, r1, r2, gate[:, :heads])
    runs = [("mma", ops.attention_prefill)] if ops.has_attention_prefill() else []
    if ops.has_attention_prefill_tc():
        runs.append(("tcgen05", ops.attention_prefill_tc))
    assert runs
    for name, run in runs:
        out = torch.zeros((n, heads * dim), dtype=dtype, device="cuda")
        run(scene.q_rows, scene.k_cache, scene.v_cache, scene.table, scene.cu_q, scene.ctx_after, out, max(scene.new),
            heads, kv_heads, dim, 64, 0.3, window, bias=table, gate=gate, gate_stride=heads + 1)
        np.testing.assert_allclose(out.double().cpu().numpy(), want, err_msg=name, **tol)
    assert int(ops.error_flag) == 0
    # one token per sequence, the context in one piece and in several
    scene = Scene(dtype, [300, 1, 70, 129, 25], [1, 1, 1, 1, 1], heads, kv_heads, dim, dim, 64, seed=dim + window + 1,
                  loud=[(0, d) for _, d in LOUD[2:]])
    gate = torch.randn(5, heads, generator=g).cuda()
    want = scene.plain(0.3, window, r1, r2, gate)
    for splits in (1, 3):
        out = torch.zeros((5, heads * dim), dtype=dtype, device="cuda")
        scratch_o = torch.empty(5 * heads * splits * dim, device="cuda")
        scratch_ml = torch.empty(5 * heads * splits * 2, device="cuda")
        ops.attention_decode(scene.q_rows, scene.k_cache, scene.v_cache, scene.table, scene.ctx_after, out, heads, kv_heads,
                             dim, 64, 0.3, window, splits, scratch_o, scratch_ml, bias=table, gate=gate, gate_stride=heads)
        np.testing.assert_allclose(out.double().cpu().numpy(), want, err_msg=f"decode in {splits}", **tol)


@pytest.mark.parametrize("window", [0, 24, 100])
@pytest.mark.parametrize("heads,kv_heads,dim", [(4, 2, 16), (2, 2, 64), (8, 1, 32), (20, 1, 64), (2, 1, 128)])
def test_fused_decode_finishes_the_new_token_itself(window, heads, kv_heads, dim):
    """Straight from the float32 rows [q | k | v | gate]: biases, the value norm, the cache write of the new token,
    attention with the bias table in one piece and in four, the gate."""
    dtype = torch.bfloat16
    ops = kernels(dtype, dim)
    assert ops.has_attention_decode_fused()
    g = torch.Generator().manual_seed(5)
    r1 = (torch.rand(heads, generator=g) + 0.1).cuda()
    r2 = (torch.rand(heads, generator=g) * 2 + 0.05).cuda()
    lengths = [300, 1, 70, 129, 25]
    scene = Scene(dtype, lengths, [1] * 5, heads, kv_heads, dim, dim, 64, seed=dim + window + 2,
                  loud=[(0, d) for _, d in LOUD[2:]])
    biases = [torch.randn(heads * dim, generator=g), torch.randn(kv_heads * dim, generator=g), torch.randn(kv_heads * dim, generator=g)]
    stride = -(-((heads + 2 * kv_heads) * dim + heads) // 8) * 8
    rows = torch.zeros(5, stride)
    eps = 1e-3
    for s, length in enumerate(lengths):
        last = length - 1
        raw_v = torch.randn(kv_heads, dim, generator=g) * 2
        finished_v = plain_zepavik.rms_divide(raw_v.double() + biases[2].double().view(kv_heads, dim), eps)
        scene.v[s][last] = finished_v.to(dtype)
        rows[s, :heads * dim] = scene.q[s][last].float().reshape(-1) - biases[0]
        rows[s, heads * dim:(heads + kv_heads) * dim] = scene.k[s][last].float().reshape(-1) - biases[1]
        rows[s, (heads + kv_heads) * dim:(heads + 2 * kv_heads) * dim] = raw_v.reshape(-1)
        page, row = scene.tables[s][last // 64], last % 64
        scene.k_cache[page, :, row] = 30.0                     # the new token is not in the cache yet
        scene.v_cache[page, :, row] = 1000.0
    gate_at = (heads + 2 * kv_heads) * dim
    rows[:, gate_at:gate_at + heads] = torch.randn(5, heads, generator=g)
    rows = rows.cuda()
    table = bias_table(r1, r2, window or 300)
    want = scene.plain(0.3, window, r1, r2, rows[:, gate_at:gate_at + heads])
    for splits in (1, 4):
        out = torch.zeros((5, heads * dim), dtype=dtype, device="cuda")
        ops.attention_decode_fused(rows, None, scene.k_cache, scene.v_cache, scene.table, scene.ctx_after, out, heads,
                                   kv_heads, dim, 64, 0.3, window, splits, True, q_bias=biases[0].cuda(),
                                   k_bias=biases[1].cuda(), v_bias=biases[2].cuda(), value_norm_eps=eps, bias=table,
                                   gate=rows[:, gate_at:], gate_stride=stride)
        np.testing.assert_allclose(out.double().cpu().numpy(), want, err_msg=f"fused decode in {splits}", rtol=2e-2, atol=2e-2)
        for s, length in enumerate(lengths):
            page, row = scene.tables[s][(length - 1) // 64], (length - 1) % 64
            np.testing.assert_allclose(scene.k_cache[page, :, row].double().cpu().numpy(), scene.k[s][length - 1].double().numpy(), rtol=1e-2, atol=1e-2)
            np.testing.assert_allclose(scene.v_cache[page, :, row].double().cpu().numpy(), scene.v[s][length - 1].double().numpy(), rtol=1e-2, atol=1e-2)


# ---- the projection that stores an activation ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 7, 16, 40, 128, 300])
def test_projection_with_an_activation_on_what_it_stores(dtype, rows):
    from stratakv_b200 import ops as _ops
    ops = kernels(dtype)
    g = torch.Generator().manual_seed(rows)
    a = torch.randn(rows, 72, generator=g).to(dtype)
    w = (torch.randn(100, 72, generator=g) * 0.3).to(dtype)
    z = a.double() @ w.double().T
    for name, want in (("relu2", torch.relu(z) ** 2), ("silu", z * torch.sigmoid(z))):
        out = torch.empty(rows, 100, dtype=dtype, device="cuda")
        ops.linear(a.cuda(), w.cuda(), out, _ops.MODE_ACT, name)
        tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=2e-2)
        np.testing.assert_allclose(out.double().cpu().numpy(), want.numpy(), err_msg=name, **tol)
    assert int(ops.error_flag) == 0
