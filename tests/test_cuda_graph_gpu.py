"""CUDA-graph decode gives the tokens and logits of eager decode (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(disable_graph: bool, forced=None):
    from mllm_b200.bench_one_batch import BenchRunner, make_synthetic_input_ids
    from mllm_b200.configs import GlobalConfig

    GlobalConfig.reset()
    cfg = GlobalConfig.get_instance()
    sc = cfg.server
    sc.model_path = "preset:qwen3-0.6b"
    sc.dtype = "bfloat16"
    sc.max_running_requests = 8
    sc.max_total_tokens = 8192
    sc.disable_cuda_graph = disable_graph
    br = BenchRunner.create(cfg, device="cuda:0")
    ids = make_synthetic_input_ids(batch_size=3, input_len=70, vocab_size=br.runner.vocab_size, seed=5)
    toks = [br.extend(ids)]
    for i in range(6):
        # with `forced`, every step is fed the other run's token, so one differing choice does not shift the rest
        toks.append(br.decode(toks[-1] if forced is None else forced[i].to(toks[-1].device)))
    torch.cuda.synchronize()
    graphs = br.runner.cuda_graph_runner
    return torch.stack([t.cpu() for t in toks]), (graphs.replays if graphs is not None else 0)


def test_graph_decode_equals_eager_decode():
    """Same inputs at every step (the graph run is fed the eager run's tokens).  The two runs are not bit-equal
    by construction: a captured step sizes the split of the KV range from the context bound, an eager step from
    the current lengths, so partial sums are added in another order; with random weights a near-tie between the
    two best logits can then fall the other way, and does so at every step while the tie lasts (random-weight
    models repeat themselves).  Two of the three requests must agree at every step, and four choices in five overall."""
    eager, n0 = _run(True)
    graph, n1 = _run(False, forced=eager)
    assert n0 == 0 and n1 == 6
    same = eager == graph
    assert same.all(0).sum().item() >= 2 and same.float().mean().item() >= 0.8, (eager, graph)


def _run_hybrid(batch: int):
    from mllm_b200.bench_one_batch import BenchRunner, make_synthetic_input_ids
    from mllm_b200.configs import GlobalConfig

    GlobalConfig.reset()
    cfg = GlobalConfig.get_instance()
    sc = cfg.server
    sc.model_path = "preset:qwen3.5-tiny"
    sc.dtype = "bfloat16"
    sc.max_running_requests = 8
    sc.max_total_tokens = 4096
    sc.context_length = 256
    br = BenchRunner.create(cfg, device="cuda:0")
    ids = make_synthetic_input_ids(batch_size=4, input_len=40, vocab_size=br.runner.vocab_size, seed=11)[:batch]
    toks = [br.extend(ids)]
    for _ in range(8):
        toks.append(br.decode(toks[-1]))
    torch.cuda.synchronize()
    graphs = br.runner.cuda_graph_runner
    return torch.stack([t.cpu() for t in toks]), graphs.replays


def test_hybrid_graph_decode_padded_row_leaves_real_requests_alone():
    """Three running requests replay the graph captured for four.  The same three requests, run next to a
    fourth real one, go through the very same captured kernels, so their tokens must be identical: the
    padded row must not touch the recurrent / convolution state of any real request (it uses the request
    table's spare row, which no request owns)."""
    three, n3 = _run_hybrid(3)
    four, n4 = _run_hybrid(4)
    assert n3 == 8 and n4 == 8
    assert torch.equal(three, four[:, :3])
