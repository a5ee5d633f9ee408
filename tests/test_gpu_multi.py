"""Fused compute+communication kernels over peer memory, on 2 GPUs of one box (child processes)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> str:
    """A TCP port that is free right now on the loopback interface (shared boxes: no fixed port numbers)."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_comm_paths_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(ROOT, "tests", "workers", "fused_comm_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert "WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("precision", ["bf16", "mxfp8"])
def test_tensor_parallel_lm_two_gpus_matches_single_process_loss(precision):
    """ParallelLm with tp = 2 on two GPUs (linears on the tcgen05 GEMMs, BF16 or block-scaled FP8): the first loss
    equals the single-process model's on the same tokens, and training steps run."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), "-m", "nexus_b200.bench.parallel", "--model", "llama2-7b", "--layers", "1",
           "--tp", "2", "--seq-len", "256", "--global-batch", "2", "--micro-batch", "1", "--precision", precision,
           "--steps", "2", "--warmup", "1", "--check"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and '"check": "first loss"' in r.stdout and "tokens/s" in r.stdout, \
        r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_llama_on_fused_kernels_matches_single_rank():
    """`models.llama_tp.LlamaTpModel` over 2 GPUs (all-gather -> GEMM and GEMM -> reduce-scatter inside the tcgen05
    kernels, vocabulary-parallel embedding and loss, fused norm exchange) against the one-rank model: loss, gradients,
    gradient norm and three optimizer steps."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(ROOT, "tests", "workers", "llama_tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert "WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm", ["fused", "nccl"])
def test_expert_parallel_moe_decoder_matches_single_rank(comm):
    """`models.moe_ep` over 2 GPUs (experts split over the ranks, rows dispatched / combined through peer memory, or
    exchanged with NCCL all-to-alls in the comparison form; fused all-reduce of the replicated gradients) against one
    rank holding all experts and sequences."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, NEXUS_B200_EP_COMM=comm)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(ROOT, "tests", "workers", "moe_ep_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert "WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("algorithm,layout", [("ring", "zigzag"), ("ring", "contiguous"), ("ulysses", "contiguous")])
def test_context_parallel_lm_two_gpus_over_peer_memory(algorithm, layout):
    """`ParallelLm` with cp = 2 on two GPUs: ring attention (the attention kernels read the other rank's K / V from
    peer memory, dK / dV slots summed by their owners) or Ulysses (head <-> sequence exchange by peer stores) inside
    every block, forward and backward.  The first loss equals the single-process model's on the same tokens and the
    training steps that follow run."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), "-m", "nexus_b200.bench.parallel", "--model", "llama2-7b", "--layers", "2",
           "--tp", "1", "--cp", "2", "--cp-algorithm", algorithm, "--cp-layout", layout, "--seq-len", "512",
           "--global-batch", "2", "--micro-batch", "1", "--steps", "2", "--warmup", "1", "--check"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and '"check": "first loss"' in r.stdout and "tokens/s" in r.stdout, \
        r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_full_shard_fsdp_two_gpus_fused_and_nccl_forms():
    """FullShard (stage 3) of the unit FSDP engine on two GPUs: parameter shards gathered by peer loads, gradients
    reduce-scattered by owner pull over symmetric memory, against the NCCL form and a single process."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", _free_port(), os.path.join(ROOT, "tests", "workers", "fsdp_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert "WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
