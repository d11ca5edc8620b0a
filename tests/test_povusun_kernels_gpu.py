"""The mechanisms of the Povusun decoder one at a time, each kernel against the plain implementation's function
(tests/plain_povusun.py): the finish of the fused projection (unit norms, the queries' temperature, a normed latent),
attention with capped scores and a gate per output number over scrambled pages, with one key made to dominate far
back, at page borders and at the query itself, the per-head projection, the recurrent unit's kernels over portions,
batches, used slots and a step that runs twice, the norm that adds a branch to the stream, the per-layer token
input, and the clamped gated unit on every projection kernel."""
import numpy as np
import pytest
import torch

import plain_povusun as plain

pytestmark = pytest.mark.gpu

F64 = torch.float64


def kernels(dtype, head_dim=16):
    from stratakv_b200 import ops
    return ops.kernels_for(dtype, head_dim, verbose=False)


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.double()
    allowed = (2e-5 if dtype == torch.float32 else 1.2e-2) * max(1.0, float(want.abs().max()))
    worst = float((got - want).abs().max())
    assert worst <= allowed, f"{what}: off by {worst:.3e} (allowed {allowed:.3e})"


def scrambled_table(n_seqs, blocks_each, generator):
    """Every sequence's pages in a random order among all pages (page 0 is left to nobody)."""
    order = (torch.randperm(n_seqs * blocks_each, generator=generator) + 1).view(n_seqs, blocks_each)
    return order.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_finish_unit_norms_temperature_and_latent(dtype):
    g = torch.Generator().manual_seed(1)
    ops = kernels(dtype)
    heads, kv_heads, dim, vdim, block = 3, 1, 20, 12, 16
    coef, every, eps = 0.5, 7, 1e-3
    positions = [0, 5, 6, 7, 12, 13, 14, 40, 41, 48]            # around the multiples of the period (p + 1 = 7, 14, 42, 49)
    n = len(positions)
    width = heads * dim + kv_heads * (dim + vdim) + 4           # (a row may be wider than its heads)
    rows = torch.randn(n, width, generator=g) * 3
    table = scrambled_table(1, 4, g)
    k_cache = torch.zeros(6, kv_heads, block, dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros(6, kv_heads, block, vdim, dtype=dtype, device="cuda")
    q_out = torch.empty(n, heads * dim, dtype=dtype, device="cuda")
    ops.qkv_finish(rows.cuda(), q_out, k_cache, v_cache, i32(positions), i32([0] * n), table.cuda(), heads, kv_heads, dim,
                   vdim, block, q_norm=True, k_norm=True, qk_norm_eps=eps, q_temperature=(coef, every))
    q = plain.unit_rms(rows[:, :heads * dim].double().view(n, heads, dim), eps)
    q = q * plain.query_temperature(torch.tensor(positions), coef, every)[:, None, None]
    close(q_out.view(n, heads, dim), q, dtype, "queries")
    k = plain.unit_rms(rows[:, heads * dim:heads * dim + dim].double().view(n, kv_heads, dim), eps)
    v = rows[:, heads * dim + dim:heads * dim + dim + vdim].double().view(n, kv_heads, vdim)
    for t, p in enumerate(positions):
        page = int(table[0, p // block])
        close(k_cache[page, :, p % block], k[t], dtype, f"key {p}")
        close(v_cache[page, :, p % block], v[t], dtype, f"value {p}")
    # rows that hold queries only (keys of another layer are used): nothing is written, the row may end after them
    k_before = k_cache.clone()
    only_q = rows[:, :heads * dim].contiguous()
    ops.qkv_finish(only_q.cuda(), q_out, k_cache, v_cache, i32(positions), i32([0] * n), table.cuda(), heads, kv_heads, dim,
                   vdim, block, write_kv=False, q_norm=True, k_norm=True, qk_norm_eps=eps)
    close(q_out.view(n, heads, dim), plain.unit_rms(only_q.double().view(n, heads, dim), eps), dtype, "queries alone")
    assert torch.equal(k_cache, k_before)
    # a latent: one "key" of its own width, normed with a weight, no values; queries pass as they are
    for rank in (40, 320):
        weight = (1.0 + torch.randn(rank, generator=g)).float()
        rows = torch.randn(n, heads * dim + rank, generator=g) * 2
        latents = torch.zeros(6, 1, block, rank, dtype=dtype, device="cuda")
        ops.qkv_finish(rows.cuda(), q_out, latents, None, i32(positions), i32([0] * n), table.cuda(), heads, 1, dim, 0, block,
                       k_norm=True, qk_norm_eps=eps, k_norm_weight=weight.cuda(), key_dim=rank)
        close(q_out, rows[:, :heads * dim], dtype, "plain queries")
        c = plain.rms_norm(rows[:, heads * dim:].double(), weight.double(), eps)
        for t, p in enumerate(positions):
            close(latents[int(table[0, p // block]), 0, p % block], c[t], dtype, f"latent {p} of {rank}")


def _attend_plain(q, k, v, scale, cap, gate):
    """q [T, H, d], k [T, G, d], v [T, G, dv], gate [T, H * dv] or None -> [T, H * dv]."""
    T, H = q.shape[0], q.shape[1]
    group = H // k.shape[1]
    scores = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(group, dim=1)) * scale
    if cap:
        scores = plain.soft_cap(scores, cap)
    out = torch.einsum("hij,jhd->ihd", plain.causal_softmax(scores), v.repeat_interleave(group, dim=1)).reshape(T, -1)
    return out * torch.sigmoid(gate) if gate is not None else out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 2, 16, 24, 5.0), (3, 3, 20, 12, 0.0), (2, 1, 64, 64, 30.0)])
def test_attention_with_a_cap_and_a_gate_per_number_finds_the_one_key(dtype, shape):
    """One key is made to dominate: far back among hundreds, at a page's last and first row, and the query's own.
    With the cap its score is the cap and the others are near zero, so a lost or shifted key moves the output."""
    heads, kv_heads, dim, vdim, cap = shape
    g = torch.Generator().manual_seed(2)
    ops = kernels(dtype)
    T, block = 330, 64
    q = torch.randn(T, heads, dim, generator=g) * 0.1
    k = torch.randn(T, kv_heads, dim, generator=g) * 0.1
    v = torch.randn(T, kv_heads, vdim, generator=g)
    gate = torch.randn(T, heads * vdim, generator=g) * 2
    marks = {329: 3, 300: 63, 301: 64, 200: 127, 201: 128, 128: 128, 64: 0, 1: 0}      # query -> the key it is to find
    for query, key in marks.items():
        direction = torch.randn(dim, generator=g)
        direction = direction / direction.norm()
        k[key, :, :] += 6.0 * direction
        q[query, :, :] = 6.0 * direction
    q, k, v = (x.to(dtype).double() for x in (q, k, v))                         # both sides see the stored values
    want = _attend_plain(q, k, v, 1.7, cap, gate.double())
    table = scrambled_table(1, 6, g)
    k_cache = torch.zeros(8, kv_heads, block, dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros(8, kv_heads, block, vdim, dtype=dtype, device="cuda")
    for t in range(T):
        k_cache[int(table[0, t // block]), :, t % block] = k[t].to(dtype).cuda()
        v_cache[int(table[0, t // block]), :, t % block] = v[t].to(dtype).cuda()
    out_width = heads * vdim + 8
    out = torch.full((T, out_width), 7.0, dtype=dtype, device="cuda")
    ops.attention_general(q.to(dtype).reshape(T, -1).cuda(), k_cache, v_cache, table.cuda(), i32(list(range(T))), i32([0] * T), out,
                          heads, kv_heads, dim, vdim, block, 1.7, gate=gate.cuda(), gate_stride=heads * vdim, softcap=cap,
                          gate_per_element=True)
    close(out[:, :heads * vdim], want, dtype, "attention")
    assert float(out[:, heads * vdim:].abs().max()) == 0.0
    for query, key in marks.items():                                            # the marked key carries the output
        alone = (v[key].repeat_interleave(heads // kv_heads, dim=0).reshape(-1) * torch.sigmoid(gate[query].double()))
        if cap == 0.0:
            close(out[query, :heads * vdim], alone, dtype, f"query {query} finds key {key}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_over_one_cache_as_keys_and_values(dtype):
    """How a cached latent is attended over: every head on the one key head, the same tensor as keys and as values,
    also wider than 256."""
    g = torch.Generator().manual_seed(3)
    ops = kernels(dtype)
    for rank in (40, 320):
        T, heads, block = 150, 3, 16
        q = (torch.randn(T, heads, rank, generator=g) * 0.3).to(dtype).double()
        c = torch.randn(T, 1, rank, generator=g).to(dtype).double()
        want = _attend_plain(q, c, c, 0.4, 0.0, None)
        table = scrambled_table(1, 10, g)
        cache = torch.zeros(12, 1, block, rank, dtype=dtype, device="cuda")
        for t in range(T):
            cache[int(table[0, t // block]), 0, t % block] = c[t, 0].to(dtype).cuda()
        out = torch.empty(T, heads * rank, dtype=dtype, device="cuda")
        ops.attention_general(q.to(dtype).reshape(T, -1).cuda(), cache, cache, table.cuda(), i32(list(range(T))), i32([0] * T),
                              out, heads, 1, rank, rank, block, 0.4)
        close(out, want, dtype, f"latent of {rank}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_headwise_projection(dtype):
    g = torch.Generator().manual_seed(4)
    ops = kernels(dtype)
    for n, heads, in_dim, out_dim, x_float, out_float in ((1, 3, 16, 16, True, True), (37, 5, 20, 44, False, False),
                                                          (70, 2, 65, 130, True, False), (33, 1, 7, 3, False, True)):
        w = (torch.randn(heads, out_dim, in_dim, generator=g) * 0.3).to(dtype)
        x_dtype = torch.float32 if x_float else dtype
        x = torch.randn(n, heads * in_dim + 3, generator=g).to(x_dtype)          # rows wider than their heads
        out = torch.full((n, heads * out_dim + 5), 9.0, dtype=torch.float32 if out_float else dtype, device="cuda")
        ops.headwise_linear(x.cuda(), w.cuda(), out, heads, zero_pad=True)
        want = torch.einsum("thi,hoi->tho", x[:, :heads * in_dim].double().view(n, heads, in_dim), w.double())
        close(out[:, :heads * out_dim], want.reshape(n, -1), dtype if not (x_float and out_float) else dtype, "product")
        assert float(out[:, heads * out_dim:].abs().max()) == 0.0


def _recurrent_tensors(width, channels, parts, taps, generator):
    part = channels // parts
    r = lambda *shape, s=0.3: torch.randn(*shape, generator=generator) * s
    return {"l0.mix.y": r(channels, width), "l0.mix.y.b": r(channels, s=0.5), "l0.mix.x": r(channels, width),
            "l0.mix.x.b": r(channels, s=0.5), "l0.mix.conv": r(channels, taps, s=0.6), "l0.mix.conv.b": r(channels, s=0.5),
            "l0.mix.ra": r(parts, part, part), "l0.mix.ra.b": r(parts, part, s=0.5), "l0.mix.ri": r(parts, part, part),
            "l0.mix.ri.b": r(parts, part, s=0.5), "l0.mix.lam": r(channels, s=0.5) - 2.5, "l0.mix.o": torch.eye(channels)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(48, 3, 3), (80, 1, 1), (64, 4, 4), (40, 5, 6)])
def test_recurrent_unit_over_portions_batches_and_used_slots(dtype, shape):
    """The unit's kernels against the plain recurrence (whose output projection is the identity here): portions
    shorter than the taps, two sequences of one step, a slot whose earlier user left its state behind, and a
    one-token step run twice."""
    channels, parts, taps = shape
    width = 24
    g = torch.Generator().manual_seed(5)
    ops = kernels(dtype)
    P = {name: t.to(dtype).double() for name, t in _recurrent_tensors(width, channels, parts, taps, g).items()}
    lengths = {"a": 23 + 300, "b": 9, "c": 12 + 130}
    inputs = {key: torch.randn(n, width, generator=g).to(dtype).double() for key, n in lengths.items()}
    want = {key: plain.rglru_mixer(h, P, "l0.", {"width": channels}) for key, h in inputs.items()}
    dev32 = lambda t: t.float().contiguous().cuda()
    w_gates = torch.cat([P["l0.mix.ra"], P["l0.mix.ri"]], dim=1).to(dtype).contiguous().cuda()
    rate = ops.rglru_rate(dev32(P["l0.mix.lam"]), torch.empty(channels, dtype=torch.float32, device="cuda"))
    slots = 4
    state = torch.full((slots + 1, (2 + taps) * channels + 3), 5.0, dtype=torch.float32, device="cuda")   # nobody's zeros
    got = {key: torch.zeros(n, channels, dtype=F64) for key, n in lengths.items()}
    done = {key: 0 for key in lengths}

    def step(parts_of_step, twice=False):
        """parts_of_step: (key, slot, count) per sequence."""
        rows, pos, seq, cu = [], [], [], [0]
        for index, (key, slot, count) in enumerate(parts_of_step):
            h = inputs[key][done[key]:done[key] + count]
            rows.append(torch.cat([h @ P["l0.mix.y"].T, h @ P["l0.mix.x"].T], dim=1))
            pos += list(range(done[key], done[key] + count)); seq += [index] * count; cu.append(cu[-1] + count)
        n = cu[-1]
        meta = (i32(pos), i32(seq), i32(cu), i32([slot for _, slot, _ in parts_of_step]))
        for _ in range(2 if twice else 1):
            yx = dev32(torch.cat(rows))
            u = torch.empty(n, channels, dtype=torch.float32, device="cuda")
            ops.rglru_conv(yx, channels, dev32(P["l0.mix.x.b"]), dev32(P["l0.mix.conv"]), dev32(P["l0.mix.conv.b"]), u, meta, state)
            gates = torch.empty(n, 2 * channels, dtype=torch.float32, device="cuda")
            ops.headwise_linear(u, w_gates, gates, parts)
            ops.rglru_gates(gates, u, yx, dev32(P["l0.mix.y.b"]), dev32(P["l0.mix.ra.b"].reshape(-1)),
                            dev32(P["l0.mix.ri.b"].reshape(-1)), rate, channels // parts)
            out = torch.empty(n, channels, dtype=dtype, device="cuda")
            longest = max(count for _, _, count in parts_of_step)
            need = ops.rglru_scan_scratch(len(parts_of_step), longest, channels)
            summary = torch.empty(need, dtype=torch.float32, device="cuda") if need else None
            ops.rglru_scan(gates, yx, channels, dev32(P["l0.mix.x.b"]), out, channels // parts, taps, meta, state, longest, summary)
        for index, (key, slot, count) in enumerate(parts_of_step):
            got[key][done[key]:done[key] + count] = out[cu[index]:cu[index + 1]].double().cpu()
            done[key] += count

    step([("a", 2, 5), ("b", 0, 1)])
    step([("b", 0, 1), ("a", 2, 1)])
    step([("a", 2, 1), ("b", 0, 1)], twice=True)
    step([("a", 2, 1)], twice=True)
    step([("a", 2, 2), ("b", 0, 6)])
    step([("a", 2, 13)])
    step([("c", 0, 1)], twice=True)                 # slot 0 again: its new user starts from nothing
    step([("c", 0, 11)])
    step([("a", 2, 300), ("c", 0, 130)])            # long enough to be walked in chunks, with unequal last chunks
    for key in lengths:
        assert done[key] == lengths[key]
        close(got[key], want[key], dtype, f"sequence {key}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_that_adds_a_branch_and_the_token_input(dtype):
    g = torch.Generator().manual_seed(6)
    ops = kernels(dtype)
    for n, hidden, dim in ((1, 64, 8), (37, 72, 5), (9, 640, 24), (301, 2048, 32)):
        x = torch.randn(n, hidden, generator=g) * 2
        y = torch.randn(n, hidden, generator=g) * 5
        gamma = 1.0 + torch.randn(hidden, generator=g) * 0.3
        following = 1.0 + torch.randn(hidden, generator=g) * 0.3
        stream = x.clone().cuda()
        ahead = torch.empty(n, hidden, dtype=dtype, device="cuda")
        ops.rmsnorm_add(y.cuda(), gamma.cuda(), 1e-4, stream, next_gamma=following.cuda(), next_eps=1e-3, next_out=ahead)
        want = x.double() + plain.rms_norm(y.double(), gamma.double(), 1e-4)
        close(stream, want, torch.float32, "stream")
        close(ahead, plain.rms_norm(want, following.double(), 1e-3), dtype, "the next norm")
        stream = x.clone().cuda()
        ops.rmsnorm_add(y.cuda(), gamma.cuda(), 1e-4, stream)
        close(stream, want, torch.float32, "stream alone")
        # the token input of layer 1 of 3
        vocab = 50
        P = {"side.embed": (torch.randn(vocab, 3 * dim, generator=g) * 2).to(dtype).double(),
             "l1.side.gate": (torch.randn(dim, hidden, generator=g) * 0.2).to(dtype).double(),
             "l1.side.proj": (torch.randn(hidden, dim, generator=g) * 0.5).to(dtype).double(), "l1.side.norm": gamma.double()}
        tokens = torch.randint(0, vocab, (n,), generator=g)
        want = plain.token_side_input(x.double(), tokens, P, "l1.", 1, dim, 1e-5)
        stream = x.clone().cuda()
        ops.token_side(stream, i32(tokens.tolist()), P["side.embed"].to(dtype).cuda(), dim, dim, P["l1.side.gate"].to(dtype).cuda(),
                       P["l1.side.proj"].to(dtype).t().contiguous().cuda(), gamma.cuda(), 1e-5, next_gamma=following.cuda(), next_eps=1e-3, next_out=ahead)
        close(stream, want, torch.float32, "stream after the token input")
        close(ahead, plain.rms_norm(want, following.double(), 1e-3), dtype, "the next norm after the token input")
        # the same with the sublayer in front still to be added: x += rmsnorm(y) * gamma first, in the same kernel
        before = x.double() + plain.rms_norm(y.double(), following.double(), 1e-4)
        want = plain.token_side_input(before, tokens, P, "l1.", 1, dim, 1e-5)
        stream = x.clone().cuda()
        ops.token_side(stream, i32(tokens.tolist()), P["side.embed"].to(dtype).cuda(), dim, dim, P["l1.side.gate"].to(dtype).cuda(),
                       P["l1.side.proj"].to(dtype).t().contiguous().cuda(), gamma.cuda(), 1e-5, next_gamma=following.cuda(),
                       next_eps=1e-3, next_out=ahead, branch=y.cuda(), post_gamma=following.cuda(), post_eps=1e-4)
        close(stream, want, torch.float32, "stream after a branch and the token input")
        close(ahead, plain.rms_norm(want, following.double(), 1e-3), dtype, "the next norm after both")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gated_unit_on_every_projection_kernel(dtype):
    """Few tokens (the weight-streaming kernel), some tens (the swapped tensor-memory kernel) and hundreds (the tiled
    ones): gate and up values beyond the limit on both sides."""
    from stratakv_b200 import ops as _ops
    from stratakv_b200.parts.ffn import pack_gate_up
    g = torch.Generator().manual_seed(7)
    ops = kernels(dtype)
    hidden, ff, limit = 128, 264, 0.75
    P = {"l0.mlp.gate": (torch.randn(ff, hidden, generator=g) * 0.15).to(dtype).double(),
         "l0.mlp.up": (torch.randn(ff, hidden, generator=g) * 0.15).to(dtype).double(), "l0.mlp.down": torch.eye(ff, dtype=F64)}
    packed = pack_gate_up(P["l0.mlp.gate"].to(dtype).cuda(), P["l0.mlp.up"].to(dtype).cuda())
    for n in (3, 16, 40, 100, 300, 2100):
        h = torch.randn(n, hidden, generator=g).to(dtype)
        want = plain.dense_feed_forward(h.double(), P, "l0.", {"limit": limit})
        assert float((h.double() @ P["l0.mlp.gate"].T).max()) > 2 * limit
        out = torch.empty(n, packed.shape[0] // 2, dtype=dtype, device="cuda")
        ops.linear(h.cuda(), packed, out, _ops.MODE_GATED, "swiglu_clamp", activation_param=limit)
        close(out[:, :ff], want, dtype, f"{n} tokens")


@pytest.mark.parametrize("head_dim", [32, 64])
def test_fused_decode_attention_finishes_the_new_token(head_dim):
    """One token a sequence, straight from the float32 projection: unit norms of the queries and the new key, the
    temperature, the cap, the gate per number; then the same for a layer that borrows its keys (rows with queries
    only, the newest key and value read from the cache)."""
    from stratakv_b200.parts.attention import fused_decode_splits
    dtype = torch.bfloat16
    ops = kernels(dtype, head_dim)
    if not ops.has_attention_decode_fused():
        pytest.skip("no fused decode kernel in this build")
    g = torch.Generator().manual_seed(8)
    heads, kv_heads, block, eps, cap, coef, every, scale = 4, 2, 16, 1e-4, 4.0, 0.5, 7, 0.3
    lengths = [130, 65, 14]                                  # positions 129, 64 and 13 are the new ones (14 = 2 * 7)
    n = len(lengths)
    q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
    table = scrambled_table(n, 9, g)
    k_cache = torch.zeros(n * 9 + 2, kv_heads, block, head_dim, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    old_k = [plain.unit_rms(torch.randn(length - 1, kv_heads, head_dim, generator=g).double(), eps).to(dtype).double() for length in lengths]
    old_v = [torch.randn(length - 1, kv_heads, head_dim, generator=g).to(dtype).double() for length in lengths]
    for s, length in enumerate(lengths):
        for t in range(length - 1):
            k_cache[int(table[s, t // block]), :, t % block] = old_k[s][t].to(dtype).cuda()
            v_cache[int(table[s, t // block]), :, t % block] = old_v[s][t].to(dtype).cuda()
    rows = torch.randn(n, q_dim + 2 * kv_dim + q_dim + 8, generator=g) * 2        # [q | k | v | gate | padding]
    gate_at = q_dim + 2 * kv_dim

    def expected(s, q_row, k_all, v_all, gate_row):
        pos = lengths[s] - 1
        q = plain.unit_rms(q_row.double().view(heads, head_dim), eps) * plain.query_temperature(torch.tensor([pos]), coef, every)
        q = q.to(dtype).double()
        scores = torch.einsum("hd,jhd->hj", q, k_all.repeat_interleave(heads // kv_heads, dim=1)) * scale
        weights = torch.softmax(plain.soft_cap(scores, cap), dim=-1)
        out = torch.einsum("hj,jhd->hd", weights, v_all.repeat_interleave(heads // kv_heads, dim=1)).reshape(-1)
        return out * torch.sigmoid(gate_row.double())

    ctx_after = i32(lengths)
    out = torch.empty(n, q_dim, dtype=dtype, device="cuda")
    splits = fused_decode_splits(n, kv_heads, max(lengths), 148)
    fused = rows.cuda()
    ops.attention_decode_fused(fused, None, k_cache, v_cache, table.cuda(), ctx_after, out, heads, kv_heads, head_dim, block,
                               scale, 0, splits, True, gate=fused[:, gate_at:], gate_stride=rows.shape[1], qk_norm_eps=eps,
                               q_temperature=(coef, every), softcap=cap, gate_per_element=True)
    new_k, new_v = [], []
    for s, length in enumerate(lengths):
        k_new = plain.unit_rms(rows[s, q_dim:q_dim + kv_dim].double().view(kv_heads, head_dim), eps).to(dtype).double()
        v_new = rows[s, q_dim + kv_dim:q_dim + 2 * kv_dim].view(kv_heads, head_dim).to(dtype).double()
        new_k.append(k_new); new_v.append(v_new)
        pos = length - 1
        close(k_cache[int(table[s, pos // block]), :, pos % block], k_new, dtype, f"cached key of sequence {s}")
        close(v_cache[int(table[s, pos // block]), :, pos % block], v_new, dtype, f"cached value of sequence {s}")
        want = expected(s, rows[s, :q_dim], torch.cat([old_k[s], k_new[None]]), torch.cat([old_v[s], v_new[None]]),
                        rows[s, gate_at:gate_at + q_dim])
        close(out[s], want, dtype, f"sequence {s}")
    # a layer that borrows these keys: rows [q | gate], nothing written
    borrowed = torch.randn(n, 2 * q_dim, generator=g) * 2
    before = k_cache.clone()
    fused = borrowed.cuda()
    ops.attention_decode_fused(fused, None, k_cache, v_cache, table.cuda(), ctx_after, out, heads, kv_heads, head_dim, block,
                               scale, 0, splits, False, gate=fused[:, q_dim:], gate_stride=2 * q_dim, qk_norm_eps=eps,
                               q_temperature=(coef, every), softcap=cap, gate_per_element=True)
    assert torch.equal(k_cache, before)
    for s in range(n):
        want = expected(s, borrowed[s, :q_dim], torch.cat([old_k[s], new_k[s][None]]), torch.cat([old_v[s], new_v[s][None]]),
                        borrowed[s, q_dim:])
        close(out[s], want, dtype, f"borrowing sequence {s}")
