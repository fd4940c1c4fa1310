"""Shared-memory metadata lane, tensor queue, the device-workspace chunk pool (on a CPU workspace) and,
on a GPU, a CUDA-IPC round trip through a child process."""
import multiprocessing as mp

import pytest
import torch

from mllm_b200.orchestrator.cuda_ipc_transport import MmItemMemoryPool, ShmSyncBuffer, unwrap_mm_inputs, wrap_mm_inputs
from mllm_b200.orchestrator.shared_memory_queue import SharedMemoryManager, TensorQueue
from mllm_b200.utils.profiling import nvtx_range, torch_profiler


def test_metadata_roundtrip_and_unlink():
    meta = {"rid": "r1", "ids": list(range(1000)), "nested": {"a": (1, 2)}}
    name = SharedMemoryManager.write_metadata("r1", meta)
    assert SharedMemoryManager.read_metadata(name) == meta
    with pytest.raises(FileNotFoundError):
        SharedMemoryManager.read_metadata(name)


def test_tensor_queue_default_mode():
    q = TensorQueue(transport_mode="default", ctx=mp.get_context("fork"))
    mm = {"pixel_values": torch.arange(12.0).view(3, 4), "image_grid_thw": torch.tensor([[1, 2, 2]]), "note": "x"}
    q.put("r7", {"prompt": "hi"}, mm)
    rid, meta, got = q.get(timeout=5)
    assert rid == "r7" and meta == {"prompt": "hi"} and got["note"] == "x"
    assert torch.equal(got["pixel_values"], mm["pixel_values"]) and got["pixel_values"].is_shared()
    q.close()
    with pytest.raises(ValueError):
        TensorQueue(transport_mode="nope")


def test_pool_chunks_recycle_and_merge():
    pool = MmItemMemoryPool(4096, device="cpu", start_recycler=False)
    a = pool.get_slice_with_flag(torch.ones(100, dtype=torch.float32))      # 400 B -> 512 B chunk
    b = pool.get_slice_with_flag(torch.full((300,), 2, dtype=torch.int16))  # 600 B -> 768 B chunk
    assert a is not None and b is not None and pool.free_bytes() == 4096 - 512 - 768
    assert torch.equal(a[0], torch.ones(100)) and a[0].data_ptr() == pool.workspace.data_ptr()
    assert pool.get_slice_with_flag(torch.zeros(4096, dtype=torch.uint8)) is None        # does not fit
    assert pool.recycle() == 0                                                          # nobody signalled yet
    f = ShmSyncBuffer.open(a[1])
    f.signal()
    f.close()
    assert pool.recycle() == 512 and pool.free_bytes() == 4096 - 768
    f = ShmSyncBuffer.open(b[1])
    f.signal()
    f.close()
    pool.recycle()
    assert pool.free_bytes() == 4096 and len(pool.free) == 1 and pool.free[0].area == (0, 4096)   # merged back
    pool.shutdown()


def test_wrap_passes_host_data_through():
    mm = {"a": torch.ones(3), "b": [1, "s", (torch.zeros(2),)]}
    w = wrap_mm_inputs(mm)
    assert w["a"] is mm["a"] and unwrap_mm_inputs(w)["b"][2][0] is mm["b"][2][0]


def test_profiling_helpers(tmp_path):
    with nvtx_range("phase"):
        pass
    with torch_profiler(False) as p:
        assert p is None
    with torch_profiler(True, activities=["CPU"], output_dir=str(tmp_path), filename_prefix="t", tag="x") as prof:
        torch.ones(10).sum()
    assert prof.exported_path.endswith(".trace.json.gz") and (tmp_path / prof.exported_path.split("/")[-1]).exists()


def _ipc_child(q_in, q_out):
    import torch as t

    from mllm_b200.orchestrator.cuda_ipc_transport import unwrap_mm_inputs as unwrap

    payload = q_in.get(timeout=60)
    got = unwrap(payload)
    q_out.put({k: v.float().sum().item() for k, v in got.items() if isinstance(v, t.Tensor)})


@pytest.mark.gpu
@pytest.mark.parametrize("use_pool", [False, True])
def test_cuda_ipc_roundtrip(use_pool):
    ctx = mp.get_context("spawn")
    q_in, q_out = ctx.Queue(), ctx.Queue()
    child = ctx.Process(target=_ipc_child, args=(q_in, q_out))
    child.start()
    pool = MmItemMemoryPool(1 << 20, device="cuda:0", start_recycler=False) if use_pool else None
    x = torch.arange(1000, device="cuda:0", dtype=torch.float32)
    payload = wrap_mm_inputs({"pixel_values": x, "grid": torch.tensor([[1, 2, 2]])}, pool=pool)
    torch.cuda.synchronize()
    q_in.put(payload)
    sums = q_out.get(timeout=120)
    child.join(timeout=30)
    assert child.exitcode == 0
    assert sums["pixel_values"] == float(x.sum()) and sums["grid"] == 5.0
    if pool is not None:
        assert pool.recycle() > 0 and pool.free_bytes() == pool.size       # the child flipped the flag
        pool.shutdown()
