"""Tensor parallelism: TP=2 gives the logits of TP=1 (gloo ranks on CPU; NCCL + fused peer-memory
kernels on GPUs).  Every rank is a child process; a rank that fails ends the run by exit code."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(world, out, device, dtype, port, extra_env=None):
    port = _free_port()      # the number passed by the test only documents the order of the runs
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE=str(world),
               NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    procs = []
    for r in range(world):
        e = dict(env, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), out, device, dtype], env=e))
    try:
        codes = [p.wait(timeout=150) for p in procs]
    except subprocess.TimeoutExpired:
        for p in procs:
            p.kill()
        raise
    assert codes == [0] * world, f"rank exit codes {codes}"
    return torch.load(out)


def test_tp2_matches_tp1_on_cpu(tmp_path):
    one = _launch(1, str(tmp_path / "tp1.pt"), "cpu", "float32", 29611)
    two = _launch(2, str(tmp_path / "tp2.pt"), "cpu", "float32", 29612)
    torch.testing.assert_close(two, one, atol=2e-4, rtol=2e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("graph", ["0", "1"])
def test_tp2_matches_tp1_on_gpu(tmp_path, graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one = _launch(1, str(tmp_path / "tp1.pt"), "cuda", "bfloat16", 29613)
    two = _launch(2, str(tmp_path / "tp2.pt"), "cuda", "bfloat16", 29614, {"TP_TEST_GRAPH": graph})
    assert (two - one).abs().max().item() < 0.15
    assert (two.argmax(-1) == one.argmax(-1)).float().mean().item() > 0.8


@pytest.mark.gpu
def test_tp2_fused_prefill_matches_nccl_on_gpu(tmp_path):
    """A prefill large enough for the sequence-sharded path (GEMM epilogue scatters tiles to the owning
    rank, reduce-scatter + add + norm + all-gather kernel, flag-gated consumer GEMM) gives the logits of
    the plain all-reduce path, for the prefill and the decode steps that follow it."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"TP_TEST_PREFILL_LEN": "256"}
    ref = _launch(2, str(tmp_path / "nccl.pt"), "cuda", "bfloat16", 29615, dict(env, TP_TEST_COMM="nccl"))
    fused = _launch(2, str(tmp_path / "fused.pt"), "cuda", "bfloat16", 29616, dict(env, TP_TEST_COMM="fused", TP_TEST_EXPECT_FUSED_PREFILL="1"))
    assert (fused - ref).abs().max().item() < 0.15
    assert (fused.argmax(-1) == ref.argmax(-1)).float().mean().item() > 0.8


@pytest.mark.parametrize("preset", ["qwen3-tiny", "qwen3-moe-tiny"])
def test_pp2_matches_single_rank_on_cpu(tmp_path, preset):
    """Two pipeline stages (gloo ranks): each builds and loads its own layers, hidden state and residual go
    from stage to stage, the last stage computes logits and shares the sampled ids; prefill and decode logits
    equal the single-rank model's."""
    env = {"TP_TEST_PRESET": preset}
    one = _launch(1, str(tmp_path / "pp1.pt"), "cpu", "float32", 29651, env)
    two = _launch(2, str(tmp_path / "pp2.pt"), "cpu", "float32", 29652, dict(env, TP_TEST_PP="2"))
    torch.testing.assert_close(two, one, atol=2e-4, rtol=2e-4)


def test_tp2_pp2_matches_single_rank_on_cpu(tmp_path):
    """Four ranks: two pipeline stages of two tensor-parallel ranks each (collective-library path)."""
    one = _launch(1, str(tmp_path / "a.pt"), "cpu", "float32", 29655)
    four = _launch(4, str(tmp_path / "b.pt"), "cpu", "float32", 29656, {"TP_TEST_PP": "2", "TP_TEST_COMM": "nccl"})
    torch.testing.assert_close(four, one, atol=3e-4, rtol=3e-4)


def test_tp2_loads_only_its_slices_from_safetensors(tmp_path):
    """Two ranks loading one safetensors file through slice handles: logits equal the single-rank model
    loaded from the same tensors, and each rank reads clearly less than the whole file (the sharded
    matrices by halves; embeddings, norms and the replicated head in full)."""
    one = _launch(1, str(tmp_path / "tp1.pt"), "cpu", "float32", 29641)
    ck = tmp_path / "ckpt"
    two = _launch(2, str(tmp_path / "tp2.pt"), "cpu", "float32", 29642, {"TP_TEST_FROM_FILES": str(ck)})
    torch.testing.assert_close(two, one, atol=2e-4, rtol=2e-4)
    for r in range(2):
        read, total = (int(x) for x in (ck / f"bytes_read_rank{r}_of2.txt").read_text().split())
        assert 0 < read < 0.85 * total, (read, total)


def test_lazy_tensor_reads_what_is_used(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    from mllm_b200.io.lazy_tensor import LazyTensor

    a = torch.arange(24.).reshape(4, 6)
    save_file({"a": a, "v": torch.arange(5)}, str(tmp_path / "t.safetensors"))
    fh = safe_open(str(tmp_path / "t.safetensors"), framework="pt", device="cpu")
    base = LazyTensor.bytes_read
    t = LazyTensor(fh.get_slice("a"), fh)
    assert tuple(t.shape) == (4, 6) and t.dim() == 2 and t.dtype == torch.float32 and t.numel() == 24
    assert LazyTensor.bytes_read == base                                  # metadata costs nothing
    assert torch.equal(t.narrow(1, 2, 2), a[:, 2:4]) and LazyTensor.bytes_read == base + 32
    assert torch.equal(t[1:3], a[1:3]) and torch.equal(t[:, :3], a[:, :3])
    p = torch.zeros(4, 6)
    p.copy_(t)                                                            # a torch function: whole tensor, once
    assert torch.equal(p, a)
    after = LazyTensor.bytes_read
    assert torch.equal(t.reshape(-1), a.reshape(-1)) and torch.equal(torch.cat([t, p], 0), torch.cat([a, a], 0))
    assert LazyTensor.bytes_read == after                                 # cached after the first full read
    v = LazyTensor(fh.get_slice("v"), fh)
    assert v.dtype == torch.int64 and int((v.float() + 1).sum()) == 15 and len(v) == 5


@pytest.mark.parametrize("kv_heads", ["2", "1"])
def test_hybrid_tp2_matches_single_rank_on_cpu(tmp_path, kv_heads):
    """Qwen3.5-style hybrid model on two gloo ranks: gated-delta-net heads (projections, convolution
    channels, gates, recurrent state) and attention heads split over the ranks, KV heads split or, when
    there is only one, replicated; prefill (chunk-parallel delta rule) and decode logits equal the
    single-rank model's."""
    env = {"TP_TEST_PRESET": "qwen3.5-tiny", "TP_TEST_KV_HEADS": kv_heads, "TP_TEST_PREFILL_LEN": "21"}
    one = _launch(1, str(tmp_path / "h1.pt"), "cpu", "float32", 29631, env)
    two = _launch(2, str(tmp_path / "h2.pt"), "cpu", "float32", 29632 + int(kv_heads), env)
    torch.testing.assert_close(two, one, atol=3e-4, rtol=3e-4)


@pytest.mark.parametrize("ep", ["0", "1"])
def test_moe_tp2_and_ep2_match_single_rank_on_cpu(tmp_path, ep):
    """Qwen3-MoE on two gloo ranks: experts sharded along their width (tensor parallel) or split between
    the ranks (expert parallel, attention stays tensor parallel); logits equal the single-rank model."""
    env = {"TP_TEST_PRESET": "qwen3-moe-tiny"}
    one = _launch(1, str(tmp_path / "moe1.pt"), "cpu", "float32", 29621, env)
    two = _launch(2, str(tmp_path / "moe2.pt"), "cpu", "float32", 29622 + int(ep), dict(env, TP_TEST_EP=ep))
    torch.testing.assert_close(two, one, atol=3e-4, rtol=3e-4)


@pytest.mark.gpu
def test_moe_ep2_matches_single_rank_on_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"TP_TEST_PRESET": "qwen3-moe-tiny"}
    one = _launch(1, str(tmp_path / "moe1.pt"), "cuda", "bfloat16", 29625, env)
    two = _launch(2, str(tmp_path / "moe2.pt"), "cuda", "bfloat16", 29626, dict(env, TP_TEST_EP="1"))
    assert (two - one).abs().max().item() < 0.2
    assert (two.argmax(-1) == one.argmax(-1)).float().mean().item() > 0.8


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_kernels_match_fp32_sums_on_n_gpus(world):
    """The fused decode reduce and the fused prefill step (GEMM with reduce-scatter epilogue -> reduce + add +
    RMSNorm + all-gather -> flag-gated consumer GEMM, three steps in a row, several tiles per CTA) on
    ``world`` GPUs against fp32 sums of the same partial products, within the rounding of the 16-bit
    partials.  Every rank is a child process; NVLS is off and the kernels use plain peer loads / stores."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m", "mllm_b200.benchmarks.tp_selftest",
           "--rows", "8192", "--k-per-rank", "512", "--steps", "3", "--deadline-s", "150"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=200, env=env, cwd=os.path.dirname(HERE))
    assert p.returncode == 0, (p.stdout[-1500:], p.stderr[-3000:])
    # one line per rank and stage (lines of different ranks may share a physical line)
    assert p.stdout.count('"stage": "canaries"') == world, p.stdout[-2000:]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [4, 8])
def test_tp_n_matches_tp1_tokens_on_gpu(tmp_path, world):
    """Token equality of the tensor-parallel model on 4 and 8 GPUs against one GPU, on a prefill long enough for
    the fused sequence-sharded path (1024 rows) and the decode steps after it."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = {"TP_TEST_PREFILL_LEN": "512", "TP_TEST_HEADS": "8"}
    one = _launch(1, str(tmp_path / "tp1.pt"), "cuda", "bfloat16", 0, env)
    many = _launch(world, str(tmp_path / "tpn.pt"), "cuda", "bfloat16", 0,
                   dict(env, TP_TEST_EXPECT_FUSED_PREFILL="1"))
    assert (many - one).abs().max().item() < 0.1
    assert torch.equal(many.argmax(-1), one.argmax(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_moe_expert_parallel_exchange_matches_single_rank_on_gpu(tmp_path, world):
    """Sparse blocks inside the fused prefill step: every rank routes the rows it owns, the rows travel to the
    ranks of their experts over peer memory, through the grouped GEMMs and back (dispatch / return kernels), and
    the logits of the prefill and of the decode steps after it equal the single-GPU model's."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = {"TP_TEST_PRESET": "qwen3-moe-tiny", "TP_TEST_PREFILL_LEN": "256"}
    one = _launch(1, str(tmp_path / "moe1.pt"), "cuda", "bfloat16", 0, env)
    many = _launch(world, str(tmp_path / "moen.pt"), "cuda", "bfloat16", 0,
                   dict(env, TP_TEST_EP="1", TP_TEST_EXPECT_FUSED_PREFILL="1", TP_TEST_EXPECT_EP_EXCHANGE="1"))
    # per (step, request) row: the layouts round differently, and a router near-tie that falls the other way sends
    # one token through another expert - such a row may differ more, but not by much and not most rows
    rows = (many - one).abs().amax(-1).flatten()
    assert (rows < 0.15).float().mean().item() >= 0.8 and rows.max().item() < 1.0, rows
    assert (many.argmax(-1) == one.argmax(-1)).float().mean().item() >= 0.8


def _rows_close(many, one, tol=0.15):
    """Per (step, request) row; with random weights a near-tie may fall the other way in one row."""
    rows = (many - one).abs().amax(-1).flatten()
    return (rows < tol).float().mean().item() >= 0.8 and rows.max().item() < 1.0


@pytest.mark.gpu
def test_pp2_matches_single_rank_on_gpu(tmp_path):
    """Two pipeline stages on two GPUs: hidden state and residual travel by NCCL send / recv, the last stage's
    sampled ids go back to the first; logits of the prefill and of the decode steps equal the single-GPU model's."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one = _launch(1, str(tmp_path / "pp1.pt"), "cuda", "bfloat16", 0)
    two = _launch(2, str(tmp_path / "pp2.pt"), "cuda", "bfloat16", 0, {"TP_TEST_PP": "2"})
    assert _rows_close(two, one), (two - one).abs().amax(-1)


@pytest.mark.gpu
def test_hybrid_tp2_matches_single_rank_on_gpu(tmp_path):
    """The Qwen3.5-style hybrid model (gated delta net + gated attention) on two GPUs: heads of both kinds split
    over the ranks, partial sums through the NCCL all-reduce; logits equal the single-GPU model's."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"TP_TEST_PRESET": "qwen3.5-tiny", "TP_TEST_KV_HEADS": "2", "TP_TEST_PREFILL_LEN": "21"}
    one = _launch(1, str(tmp_path / "h1.pt"), "cuda", "bfloat16", 0, env)
    two = _launch(2, str(tmp_path / "h2.pt"), "cuda", "bfloat16", 0, env)
    assert _rows_close(two, one), (two - one).abs().amax(-1)
