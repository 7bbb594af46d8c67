"""Replayed launch sequences: one CUDA graph, captured once under a replay reservation, serves steps whose batches
differ in request count, positions, query-run lengths and in which kernels have work (the reference records one
replay program per bucket and rewrites its scalar parameters per submission:
crates/inference-backend-metal/src/metal/stream, crates/inference-executor-core/src/replay.rs)."""
import numpy as np
import pytest

import checks
import gpuharness as G
from oracle import psi_oracle as O

pkg = G.pkg
pytestmark = pytest.mark.gpu

CAPACITY = 64   # num_total_tokens of every step: the recorded bucket
BATCHES = [
    # (req_slots, first positions, query-run lengths)
    ([0, 1, 2, 3, 4], [100, 257, 31, 640, 5], [1, 1, 1, 1, 1]),
    ([5, 2, 7], [12, 300, 999], [2, 1, 4]),
    ([1, 6, 3], [700, 90, 40], [48, 1, 1]),          # a long query run: the chunk kernel has work
    ([4], [512], [64]),                               # only a long run: the decode kernel has none
    ([0, 1, 2, 3, 4, 5, 6, 7], [1, 2, 3, 4, 5, 6, 7, 8], [1] * 8),
]


@pytest.fixture
def side_stream():
    """The legacy default stream cannot be captured: the rig (which adopts torch's current stream) and the torch
    work around it run on a stream of their own."""
    import torch
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        yield stream
    torch.cuda.synchronize()


def test_the_default_stream_is_refused():
    rig = G.Rig(pkg.BF16, 8, 2, 128, 16, 0.1, (2, 1, 8, 1), 16, num_pages=16)
    with pytest.raises(pkg.PsiError, match="legacy default stream"):
        rig.ctx.capture_begin()
    rig.close()


@pytest.mark.parametrize("kernel_mode", [pkg.KERNEL_MMA, pkg.KERNEL_GENERIC])
def test_one_captured_graph_serves_changing_batches(kernel_mode, side_stream):
    import torch
    hq, hkv, d, p = 16, 2, 128, 16
    scale = 1.0 / np.sqrt(d)
    rig = G.Rig(pkg.BF16, hq, hkv, d, p, float(scale), (8, 1, 80, 1), CAPACITY, num_pages=700, kernel_mode=kernel_mode)
    gen = torch.Generator(device="cuda").manual_seed(17)
    rig.arena.copy_((torch.randn(rig.arena.shape, device="cuda", generator=gen) * 0.5).to(torch.bfloat16))
    ids = np.random.default_rng(4).permutation(700).astype(np.uint32)
    for slot in range(8):
        rig.set_pages(slot, 0, ids[slot * 80:(slot + 1) * 80])
    q = torch.zeros((CAPACITY, hq, d), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((CAPACITY, hkv, d), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    out = torch.zeros_like(q)
    rig.gqa.reserve_replay()

    def load(batch, seed):
        slots, starts, runs = batch
        t = sum(runs)
        g2 = torch.Generator(device="cuda").manual_seed(seed)
        q[:t] = torch.randn((t, hq, d), device="cuda", generator=g2).to(torch.bfloat16)
        k[:t] = (torch.randn((t, hkv, d), device="cuda", generator=g2) * 0.5).to(torch.bfloat16)
        v[:t] = (torch.randn((t, hkv, d), device="cuda", generator=g2) * 0.5).to(torch.bfloat16)
        cu = np.concatenate([[0], np.cumsum(runs)]).astype(np.uint32)
        shape = rig.gqa.prepare_bucketed_with_token_capacity(slots, starts, cu, CAPACITY)
        assert shape.num_total_tokens == CAPACITY and shape.num_tokens == t
        return t

    # record once, on the first batch (an eager step first: kernels configure themselves outside the capture)
    load(BATCHES[0], 0)
    rig.gqa.append_attend(rig.pages, rig.table, 0, k, v, q, out)
    rig.ctx.sync()
    rig.ctx.capture_begin()
    with pytest.raises(pkg.PsiError, match="stays outside captured graphs"):
        rig.gqa.prepare([0], [1], [0, 1])
    rig.gqa.append_attend(rig.pages, rig.table, 0, k, v, q, out)
    graph = rig.ctx.capture_end()
    assert graph.kernel_count() >= 3   # append, map and chunk (and the generic kernel's reduce) are always present

    for index, batch in enumerate(BATCHES):
        t = load(batch, 100 + index)
        before = rig.arena.clone()
        out.fill_(7.0)
        rig.gqa.append_attend(rig.pages, rig.table, 0, k, v, q, out)   # the same launches, eagerly
        rig.ctx.sync()
        eager_out, eager_arena = out.clone(), rig.arena.clone()
        rig.arena.copy_(before)
        out.fill_(7.0)
        graph.launch()
        rig.ctx.sync()
        assert torch.equal(out.view(torch.int16), eager_out.view(torch.int16)), index
        assert torch.equal(rig.arena.view(torch.int16), eager_arena.view(torch.int16)), index
        assert torch.all(out[t:] == 7.0)   # rows beyond the active tokens are not written
        # and the step is right: against the oracle on the arena after the append
        slots, positions = G.flat_metadata(batch[0], batch[1], np.concatenate([[0], np.cumsum(batch[2])]))
        want = rig.oracle_attention(q[:t], slots, positions)
        got = O.decode(checks.to_numpy_bits(out[:t]), O.BF16)
        assert np.abs(got - want.reshape(got.shape)).max() <= 2e-2, index
        assert rig.gqa.device_status() == 0
    graph.close()
    rig.close()


def test_capture_refuses_buffers_that_would_grow(side_stream):
    import torch
    rig = G.Rig(pkg.BF16, 8, 2, 128, 16, 0.1, (2, 1, 8, 1), 16, num_pages=16)
    for slot in range(2):
        rig.set_pages(slot, 0, np.arange(slot * 8, slot * 8 + 8, dtype=np.uint32))
    q = torch.zeros((16, 8, 128), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    o = torch.zeros((16, 8, 128), dtype=torch.float32, device="cuda")
    rig.gqa.prepare([0, 1], [3, 5], [0, 1, 2])
    rig.ctx.capture_begin()
    # the combine path allocates its pointer table on first use: refused inside a capture instead of breaking it
    m = torch.zeros((16, 8), dtype=torch.float32, device="cuda")
    with pytest.raises(pkg.PsiError, match="grow during stream capture"):
        rig.gqa.combine([o], [m], [m], 2, out)
    graph = rig.ctx.capture_end()
    graph.close()
    rig.close()
