"""GPU parity of the stages the reference records next to the path and this library fuses into it: q/k RMSNorm + RoPE
with the KV page write (one launch), and the sigmoid gate in the attention epilogue."""
import math

import numpy as np
import pytest

import checks
import gpuharness as G
import workloads as W
from oracle import psi_oracle as O

pkg = G.pkg
pytestmark = pytest.mark.gpu


def test_bf16_norm_rounding_order_is_bit_exact_for_q_and_k():
    # crates/inference-backend-metal/src/components/rms_norm_rope.rs:476-519 through the fused launch
    import torch
    x = O.encode(np.array([0.73046875, -1.171875, 0.43945313, 2.03125], dtype=np.float32), O.BF16)
    w = O.encode(np.array([1.296875, 0.8984375, 1.1015625, 0.703125], dtype=np.float32), O.BF16)
    rig = G.Rig(pkg.BF16, 1, 1, 4, 2, 0.5, (1, 1, 1, 1), 1, num_pages=1)
    rig.set_pages(0, 0, [0])
    rig.gqa.set_norm_rope(pkg.NormRopeConfig(2, 1e-6, 1_000_000.0, 0, 1, 1, 1, 1, 1, 0), w.tolist(), w.tolist())
    rig.gqa.prepare([0], [0], [0, 1])
    xin = torch.from_numpy(x.view(np.int16).copy()).cuda().view(torch.bfloat16).reshape(1, 1, 4)
    q_out = torch.zeros_like(xin)
    rig.gqa.norm_rope_append(rig.pages, rig.table, 0, xin, xin, xin, q_out)
    rig.ctx.sync()
    inv, factor, _, _ = O.rope_parameters(2, 1_000_000.0)
    expected = O.rms_norm_rope(x, O.BF16, w, [0], 1, 4, 2, 1e-6, inv, factor)
    assert G.bits_of(q_out).reshape(-1).tolist() == expected.tolist()
    arena = rig.arena_bits()       # page = [K: 2 tokens x 4][V: 2 tokens x 4]; token 0
    assert arena[:4].tolist() == expected.tolist() and arena[8:12].tolist() == x.tolist()
    rig.close()


def test_f32_yarn_rotation_at_long_context():
    # rms_norm_rope.rs:414-474: position 262,143, tolerance 1e-3 against the CPU expectation
    import torch
    factor = float(np.float32(1.0) + np.float32(0.1) * np.log(np.float32(32.0)))
    x = np.array([((i * 37 % 29) - 14.0) / 8.0 for i in range(128)], dtype=np.float32)
    w = O.encode(np.array([0.75 + (i % 11) / 20.0 for i in range(128)], dtype=np.float32), O.BF16)
    blocks = 262144 // 16
    rig = G.Rig(pkg.F32, 1, 1, 128, 16, 0.1, (1, 1, blocks, 1), 1, num_pages=1)
    rig.gqa.set_norm_rope(pkg.NormRopeConfig(128, 1e-6, 10_000_000.0, 1, 32.0, factor, 32.0, 1.0, 8192, 1), w.tolist(),
                          w.tolist())
    rig.gqa.prepare([0], [262143], [0, 1])
    xin = torch.from_numpy(x.copy()).cuda().reshape(1, 1, 128)
    q_out = torch.zeros_like(xin)
    rig.gqa.norm_rope_append(rig.pages, rig.table, 0, xin, xin, xin, q_out)
    rig.ctx.sync()
    inv, f, _, _ = O.rope_parameters(128, 10_000_000.0, O.Yarn(1, 32.0, factor, 32.0, 1.0, 8192, 1))
    expected = O.rms_norm_rope(x, O.F32, w, [262143], 1, 128, 128, 1e-6, inv, f)
    assert np.max(np.abs(q_out.cpu().numpy().reshape(-1) - expected)) < 1e-3
    rig.close()


@pytest.mark.parametrize("dtype,head_dim,rope_dim", [(pkg.BF16, 256, 64), (pkg.BF16, 128, 128), (pkg.F16, 128, 64),
                                                     (pkg.F32, 64, 32)])
def test_fused_norm_rope_append_then_attention_matches_the_staged_oracle(dtype, head_dim, rope_dim):
    import torch
    rng = np.random.default_rng(head_dim + rope_dim)
    spec = W.Spec("norm-rope", dtype, 8, 2, head_dim, 16, [300, 41, 0, 1000], [3, 1, 20, 2], seed=21)
    s = W.Session(spec)
    wq = O.encode(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32), O.BF16)
    wk = O.encode(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32), O.BF16)
    cfg = pkg.NormRopeConfig(rope_dim, 1e-6, 1_000_000.0, 0, 1, 1, 1, 1, 1, 0)
    s.gqa.set_norm_rope(cfg, wq.tolist(), wk.tolist())
    q_raw, k_raw = s.q.clone(), s.k.clone()
    before = checks.to_numpy_bits(s.arena)
    s.gqa.norm_rope_append(s.pages, s.table, 0, q_raw, k_raw, s.v, s.q)     # s.q now holds the normalised queries
    s.attend()
    s.ctx.sync()
    # oracle: the same three stages one after the other
    positions = [int(c) + j for c, n in zip(spec.context_lens, spec.q_len) for j in range(int(n))]
    inv, factor, _, _ = O.rope_parameters(rope_dim, 1_000_000.0)
    q_ref = O.rms_norm_rope(checks.to_numpy_bits(q_raw), dtype, wq, positions, spec.num_q_heads, head_dim, rope_dim,
                            1e-6, inv, factor)
    k_ref = O.rms_norm_rope(checks.to_numpy_bits(k_raw), dtype, wk, positions, spec.num_kv_heads, head_dim, rope_dim,
                            1e-6, inv, factor)
    ulp = 2.0 ** -7 if dtype == pkg.BF16 else (2.0 ** -10 if dtype == pkg.F16 else 1e-5)
    q_got = O.decode(checks.to_numpy_bits(s.q), dtype)
    q_exp = O.decode(q_ref, dtype)
    assert np.max(np.abs(q_got - q_exp) / np.maximum(1.0, np.abs(q_exp))) <= 2 * ulp     # sin/cos differ by an ulp at most
    if dtype != pkg.F32:   # f32 keeps every bit of the row sum, whose summation order differs between the two sides
        assert np.mean(checks.to_numpy_bits(s.q) == q_ref) > 0.98
    # pages: the oracle's page write of its own normalised keys, compared through the decoded values
    s2_k = s.k.clone()
    s.k.copy_(G.to_device(O.decode(k_ref, dtype), dtype).reshape(s.k.shape))
    expected_arena = checks.expected_arena_after_append(s, before)
    s.k.copy_(s2_k)
    got_arena = checks.to_numpy_bits(s.arena).reshape(-1)
    diff = np.abs(O.decode(got_arena, dtype) - O.decode(expected_arena, dtype))
    assert np.max(diff / np.maximum(1.0, np.abs(O.decode(expected_arena, dtype)))) <= 2 * ulp
    if dtype != pkg.F32:
        assert np.mean(got_arena == expected_arena) > 0.9999  # everything but a few rotated elements is bit-identical
    # attention over the pages the GPU wrote, with the GPU's normalised queries, against the oracle
    checks.assert_attention_close(s)
    s.close()


@pytest.mark.parametrize("dtype,head_dim,gated", [(pkg.BF16, 256, True), (pkg.BF16, 128, False), (pkg.F16, 128, True),
                                                  (pkg.F32, 64, True)])
def test_projection_layout_front_stage_equals_split_then_norm_rope_append(dtype, head_dim, gated):
    # The de-interleave of the fused projection (GQAQGKVSplitKernel / GQAQKVSplitKernel) folded into the front-stage
    # launch: reading q, k, v in place from [T][width] must give exactly what the split followed by
    # psi_gqa_norm_rope_append gives - same kernel arithmetic, only the source addresses differ - and the gate rows
    # must come out as a bit copy.  The split itself is the oracle's, pinned to the reference's vector.
    import torch
    rng = np.random.default_rng(head_dim + int(gated))
    spec = W.Spec("projection", dtype, 8, 2, head_dim, 16, [300, 41, 0, 1000], [3, 1, 20, 2], seed=23)
    a, b = W.Session(spec), W.Session(spec)
    wq = O.encode(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32), O.BF16)
    wk = O.encode(1.0 + 0.1 * rng.standard_normal(head_dim).astype(np.float32), O.BF16)
    cfg = pkg.NormRopeConfig(64 if head_dim > 64 else 32, 1e-6, 1_000_000.0, 0, 1, 1, 1, 1, 1, 0)
    t, hq, hkv = spec.num_tokens, spec.num_q_heads, spec.num_kv_heads
    width = (2 if gated else 1) * hq * head_dim + 2 * hkv * head_dim
    projection = torch.randn((t, width), device=a.device).to(a.tdtype)
    q_bits, g_bits, k_bits, v_bits = O.projection_split(checks.to_numpy_bits(projection), dtype, gated, t, hq, hkv,
                                                        head_dim)
    as_device = lambda bits, like: torch.from_numpy(bits.view(np.int16) if dtype != pkg.F32 else bits).to(a.device) \
        .view(like.dtype).reshape(like.shape)
    # staged: split on the host, then the contiguous front stage
    a.gqa.set_norm_rope(cfg, wq.tolist(), wk.tolist())
    q_a = torch.zeros_like(a.q)
    a.gqa.norm_rope_append(a.pages, a.table, 0, as_device(q_bits, a.q), as_device(k_bits, a.k), as_device(v_bits, a.v),
                           q_a)
    a.ctx.sync()
    # fused: the projection as it is
    b.gqa.set_norm_rope(cfg, wq.tolist(), wk.tolist())
    q_b = torch.zeros_like(b.q)
    gates = torch.full_like(b.q, 7.0) if gated else None
    b.gqa.projection_norm_rope_append(b.pages, b.table, 0, projection, gated, q_b, gates)
    b.ctx.sync()
    assert np.array_equal(checks.to_numpy_bits(q_a), checks.to_numpy_bits(q_b))
    assert np.array_equal(checks.to_numpy_bits(a.arena), checks.to_numpy_bits(b.arena))
    if gated:
        assert np.array_equal(checks.to_numpy_bits(gates).reshape(-1), g_bits.reshape(-1))
    # the V rows are in their pages bit for bit: gather the appended positions of the longest request
    seq = int(np.argmax(spec.context_lens))
    cu = np.concatenate([[0], np.cumsum(spec.q_len)])
    lo, n = int(spec.context_lens[seq]), int(spec.q_len[seq])
    kout = torch.zeros((n, hkv, head_dim), dtype=b.tdtype, device=b.device)
    vout = torch.zeros_like(kout)
    b.gqa.page_gather(b.pages, b.table, seq, 0, lo, lo + n, kout, vout)
    b.ctx.sync()
    assert np.array_equal(checks.to_numpy_bits(vout), v_bits[cu[seq]:cu[seq] + n])
    # and the attention over those pages with those queries against the oracle
    b.q.copy_(q_b)
    b.attend()
    b.ctx.sync()
    checks.assert_attention_close(b)
    if not gated:   # a gated profile without gates_out is refused before any launch
        b.close()
        a.close()
        return
    with pytest.raises(pkg.PsiError, match="needs gates_out"):
        b.gqa.projection_norm_rope_append(b.pages, b.table, 0, projection, True, q_b, None)
    a.close()
    b.close()


@pytest.mark.parametrize("index,scale_down,kernel_mode", [(2, 8, pkg.KERNEL_AUTO), (5, 64, pkg.KERNEL_AUTO),
                                                          (3, 16, pkg.KERNEL_GENERIC)])
def test_gate_fused_into_the_attention_epilogue(index, scale_down, kernel_mode):
    import torch
    s = W.Session(W.config(index, scale_down=scale_down), kernel_mode=kernel_mode)
    s.append()
    gates = (2.0 * torch.randn(s.q.shape, device=s.device)).to(s.tdtype)
    s.attend()
    s.ctx.sync()
    plain = checks.to_numpy_bits(s.out)
    s.gqa.attend_gated(s.pages, s.table, 0, s.q, gates, s.out)
    s.ctx.sync()
    expected = O.decode(O.activation_gate(plain, checks.to_numpy_bits(gates), s.spec.dtype), s.spec.dtype)
    got = O.decode(checks.to_numpy_bits(s.out), s.spec.dtype)
    diff = np.abs(got - expected)
    assert diff.max() <= 2e-2 and diff.mean() <= 2e-3, (diff.max(), diff.mean())
    # and against the f32 oracle attention gated in f64
    attn, rows = checks.oracle_attention(s)
    g64 = O.decode(checks.to_numpy_bits(gates), s.spec.dtype).astype(np.float64)[rows]
    exact = attn.astype(np.float64) / (1.0 + np.exp(-g64))
    assert np.abs(got[rows] - exact).max() <= 2e-2
    s.close()


@pytest.mark.parametrize("dtype,tol", [(pkg.F32, 1e-5), (pkg.BF16, 1e-2)])
def test_block_partial_matches_the_reference_vectors(dtype, tol):
    # GQABlockSDPAKernel (crates/inference-backend-metal/src/components/gqa_block_attention_test.rs:23-139): block 3,
    # 5 q heads over one KV head, head_dim 32, 6 tokens of ramp inputs; tolerances are the reference's
    import torch
    block, hq, hkv, d, t = 3, 5, 1, 32, 6
    scale = float(np.float32(1.0) / np.sqrt(np.float32(32.0)))
    q = O.encode(np.arange(t * hq * d, dtype=np.float32) * np.float32(0.03125) - np.float32(0.4), dtype)
    k = O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(-0.025) + np.float32(0.3), dtype)
    v = O.encode(np.arange(t * hkv * d, dtype=np.float32) * np.float32(0.05) - np.float32(0.2), dtype)
    want_o, want_m, want_l = O.block_sdpa(q, k, v, dtype, t, block, hq, hkv, d, scale)
    rig = G.Rig(dtype, hq, hkv, d, 16, scale, (1, 1, 1, 1), 8, num_pages=1)
    dq, dk, dv = (G.bits_to_device(x, dtype) for x in (q, k, v))
    slots = torch.tensor([5, 4, 3, 2, 1, 0], dtype=torch.int32, device="cuda")   # partial slots in reverse order
    o = torch.full((8, hq, d), 7.0, dtype=torch.float32, device="cuda")
    m = torch.full((8, hq), 7.0, dtype=torch.float32, device="cuda")
    l = torch.full((8, hq), 7.0, dtype=torch.float32, device="cuda")
    rig.gqa.block_partial(dq, dk, dv, t, block, o, m, l, slot_indices=slots)
    rig.ctx.sync()
    got_o, got_m, got_l = (x.cpu().numpy() for x in (o, m, l))
    for token in range(t):
        assert np.abs(got_o[5 - token] - want_o[token]).max() < tol
        assert np.abs(got_m[5 - token] - want_m[token]).max() < 1e-4
        assert np.abs(got_l[5 - token] - want_l[token]).max() < 1e-4
    assert np.all(got_o[6:] == 7.0) and np.all(got_m[6:] == 7.0)  # slots nobody was given stay untouched
    with pytest.raises(pkg.PsiError, match="complete request blocks"):
        rig.gqa.block_partial(dq, dk, dv, 5, block, o, m, l)
    rig.close()


def test_history_plus_block_composite():
    # The DSpark composite: every draft token attends to the request's whole paged history (no causal cut inside the
    # block) and, bidirectionally, to the tokens of its own draft block; history partial + block partial -> combine.
    import torch
    hq, hkv, d, p, block = 16, 2, 128, 16, 4
    ctx = [300, 77]                                  # history tokens of two requests, one draft block each
    scale = 1.0 / np.sqrt(d)
    rig = G.Rig(pkg.BF16, hq, hkv, d, p, float(scale), (2, 1, 32, 1), 16, num_pages=64)
    gen = torch.Generator(device="cuda").manual_seed(21)
    rig.arena.copy_((torch.randn(rig.arena.shape, device="cuda", generator=gen) * 0.5).to(torch.bfloat16))
    rng = np.random.default_rng(3)
    ids = rng.permutation(64).astype(np.uint32)
    rig.set_pages(0, 0, ids[:32])
    rig.set_pages(1, 0, ids[32:])
    t = 2 * block
    q = (torch.randn((t, hq, d), device="cuda", generator=gen)).to(torch.bfloat16)
    lk = (torch.randn((t, hkv, d), device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    lv = (torch.randn((t, hkv, d), device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    # history partial: each draft token is a one-token "request" at the last history position, so it sees [0, ctx)
    req_slots = [0] * block + [1] * block
    positions = [ctx[0] - 1] * block + [ctx[1] - 1] * block
    rig.gqa.prepare(req_slots, positions, list(range(t + 1)))
    parts = []
    for _ in range(2):
        parts.append((torch.zeros((t, hq, d), dtype=torch.float32, device="cuda"),
                      torch.zeros((t, hq), dtype=torch.float32, device="cuda"),
                      torch.zeros((t, hq), dtype=torch.float32, device="cuda")))
    rig.gqa.attend_partial(rig.pages, rig.table, 0, q, *parts[0])
    rig.gqa.block_partial(q, lk, lv, t, block, *parts[1])
    out = torch.zeros_like(q)
    rig.gqa.combine([x[0] for x in parts], [x[1] for x in parts], [x[2] for x in parts], t, out)
    rig.ctx.sync()
    # expectation: one exact softmax over history keys followed by the block's keys, in float64
    arena = O.decode(checks.to_numpy_bits(rig.arena), O.BF16).astype(np.float64).reshape(64, 2, hkv, p, d)
    qf = O.decode(checks.to_numpy_bits(q), O.BF16).astype(np.float64)
    kf = O.decode(checks.to_numpy_bits(lk), O.BF16).astype(np.float64)
    vf = O.decode(checks.to_numpy_bits(lv), O.BF16).astype(np.float64)
    got = O.decode(checks.to_numpy_bits(out), O.BF16)
    worst = 0.0
    for token in range(t):
        r = token // block
        pages = rig.table_host[r, 0].reshape(-1)
        for head in range(hq):
            kvh = head // (hq // hkv)
            hist_k = np.concatenate([arena[pages[i], 0, kvh] for i in range(-(-ctx[r] // p))])[:ctx[r]]
            hist_v = np.concatenate([arena[pages[i], 1, kvh] for i in range(-(-ctx[r] // p))])[:ctx[r]]
            keys = np.concatenate([hist_k, kf[r * block:(r + 1) * block, kvh]])
            values = np.concatenate([hist_v, vf[r * block:(r + 1) * block, kvh]])
            scores = keys @ qf[token, head] * scale
            w = np.exp(scores - scores.max())
            want = w @ values / w.sum()
            worst = max(worst, np.abs(got[token, head] - want).max())
    assert worst <= 2e-2, worst
    rig.close()


def test_read_bandwidth_probe_reports_a_plausible_figure():
    """The read-only probe streams a buffer larger than L2 and reports HBM-scale bandwidth; bad sizes are refused."""
    ctx = pkg.Context(0)
    gbs = ctx.read_bandwidth(1 << 30, 3)
    assert 1000.0 < gbs < 12000.0, gbs
    with pytest.raises(pkg.PsiError):
        ctx.read_bandwidth(8, 1)
    ctx.close()
