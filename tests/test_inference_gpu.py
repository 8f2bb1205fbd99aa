"""Paged KV cache kernels and the inference engine."""
import os
import subprocess
import sys

import pytest
import torch

from ferrotorch_b200 import _native
from ferrotorch_b200.nn.paged import OutOfPages, PagedAttentionManager, PagedKVCache
from ferrotorch_b200.ops import reference as R

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.parametrize("D,Hq,Hkv,splits", [(128, 8, 2, 1), (128, 8, 2, 3), (64, 4, 4, 2), (128, 4, 1, 0)])
def test_paged_decode_matches_reference(D, Hq, Hkv, splits):
    torch.manual_seed(D + Hq + splits)
    B, bs = 5, 16
    lens = [1, 17, 64, 100, 333]
    cache = PagedKVCache(1, Hkv, D, num_blocks=64, max_seqs=B, max_seq_len=512, block_size=bs)
    mgr = PagedAttentionManager(cache)
    ks, vs = [], []
    for b, n in enumerate(lens):
        assert mgr.add_sequence(n) == b
        k = torch.randn(n, Hkv, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(n, Hkv, D, device="cuda").to(torch.bfloat16)
        ks.append(k), vs.append(v)
        pos = torch.arange(n, device="cuda", dtype=torch.int32)
        sid = torch.full((n,), b, device="cuda", dtype=torch.int32)
        cache.append(0, k, v, pos, sid)
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    out = cache.decode(0, q, torch.tensor(lens, device="cuda", dtype=torch.int32), n_splits=splits)
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        gk, gv = cache.gather(0, b, n)
        assert torch.equal(gk, ks[b]) and torch.equal(gv, vs[b])
        want, _ = R.attention(q[b][None, None], ks[b][None], vs[b][None], causal=False)
        err = (out[b].float() - want[0, 0].float()).abs().max().item()
        assert err < 2e-2, "seq %d len %d err %g" % (b, n, err)


@pytest.mark.gpu
@pytest.mark.parametrize("Hq,Hkv,splits,bs", [(8, 8, 2, 16), (8, 4, 1, 32), (16, 2, 4, 16), (32, 8, 0, 8), (8, 2, 2, 128)])
def test_paged_decode_tensor_core_kernel_long_contexts(Hq, Hkv, splits, bs):
    # head_dim 128 with a page size dividing 128 takes the tcgen05 kernel: group sizes 1 / 2 / 4 / 8,
    # contexts long enough to wrap its three-stage ring several times, growing score maxima
    # (lazy rescale of the accumulator), tails that end inside a page and inside a tile
    torch.manual_seed(Hq + Hkv + splits + bs)
    D = 128
    lens = [1, 127, 129, 700, 1531]
    B = len(lens)
    cache = PagedKVCache(1, Hkv, D, num_blocks=sum((n + bs - 1) // bs for n in lens) + 4, max_seqs=B,
                         max_seq_len=2048, block_size=bs)
    mgr = PagedAttentionManager(cache)
    ks, vs = [], []
    for b, n in enumerate(lens):
        assert mgr.add_sequence(n) == b
        ramp = torch.linspace(0.3, 2.5, n, device="cuda").view(n, 1, 1)
        k = (torch.randn(n, Hkv, D, device="cuda") * ramp).to(torch.bfloat16)
        v = torch.randn(n, Hkv, D, device="cuda").to(torch.bfloat16)
        ks.append(k), vs.append(v)
        cache.append(0, k, v, torch.arange(n, device="cuda", dtype=torch.int32),
                     torch.full((n,), b, device="cuda", dtype=torch.int32))
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    out = cache.decode(0, q, torch.tensor(lens, device="cuda", dtype=torch.int32), n_splits=splits)
    torch.cuda.synchronize()
    assert _native.device_status(0) == 0
    for b, n in enumerate(lens):
        want, _ = R.attention(q[b][None, None], ks[b][None], vs[b][None], causal=False)
        err = (out[b].float() - want[0, 0].float()).abs().max().item()
        assert err < 3e-2, "seq %d len %d err %g" % (b, n, err)


def test_page_pool_bookkeeping():
    cache = PagedKVCache(1, 1, 8, num_blocks=4, max_seqs=2, max_seq_len=64, block_size=16, device="cpu",
                         dtype=torch.float32)
    mgr = PagedAttentionManager(cache)
    a = mgr.add_sequence(20)            # 2 pages
    assert mgr.free_pages == 2
    b = mgr.add_sequence(16)            # 1 page
    mgr.extend(b, 1)                    # 17 tokens -> 2 pages
    assert mgr.free_pages == 0
    with pytest.raises(OutOfPages):
        mgr.extend(a, 20)
    assert mgr.num_sequences() == 2 and mgr.pool_utilization() == 1.0 and mgr.pool().num_used == 4 == mgr.pool().num_total
    mgr.remove_sequence(a)
    assert mgr.free_pages == 2 and a not in mgr.active and mgr.pool_utilization() == 0.5
    k = torch.arange(17 * 8, dtype=torch.float32).view(17, 1, 8)
    cache.append(0, k, -k, torch.arange(17, dtype=torch.int32), torch.full((17,), b, dtype=torch.int32))
    gk, gv = cache.gather(0, b, 17)
    assert torch.equal(gk, k) and torch.equal(gv, -k)
    out = cache.decode(0, torch.ones(2, 1, 8), torch.tensor([0, 17], dtype=torch.int32))
    assert out.shape == (2, 1, 8)


def _run(nproc, port, graph=False, weights="bf16"):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", FT_TEST_GRAPH="1" if graph else "0",
               FT_COMM_TIMEOUT_MS="5000", FT_TEST_WEIGHTS=weights)
    script = os.path.join(HERE, "engine_worker.py")
    cmd = [sys.executable, script] if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
        "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout


@pytest.mark.gpu
def test_engine_single_gpu():
    _run(1, 0)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_engine_tensor_parallel_2():
    _run(2, 29551)


@pytest.mark.gpu
def test_engine_single_gpu_cuda_graph():
    _run(1, 0, graph=True)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_engine_tensor_parallel_2_cuda_graph():
    _run(2, 29552, graph=True)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_engine_tensor_parallel_all_gpus_cuda_graph():
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    if n == 2:
        pytest.skip("covered by the two-GPU test")
    _run(n, 29553, graph=True)


# The Q4_0 weight format of the engine is a composition of kernels that each have their own test
# (gather, dequant-GEMM); these two check the composition.


@pytest.mark.gpu
def test_engine_q4_0_single_gpu():
    _run(1, 0, weights="q4_0")


@pytest.mark.gpu
@pytest.mark.multigpu
def test_engine_q4_0_tensor_parallel_2():
    _run(2, 29553, weights="q4_0")
