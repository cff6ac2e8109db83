"""Failure detection, exercised on the host only: dead worker ranks, dead DP replicas, broken
checkpoints. Nothing here touches a GPU."""
import os
import signal
import struct
import time

import pytest
import torch

from xixi_vllm_b200 import Engine, EngineConfig, SamplingParams
from xixi_vllm_b200.models.loader import SafetensorsSource, write_safetensors


def _cfg(model_dir, **kw):
    base = dict(device="cpu", dtype="float32", num_kvcache_blocks=64, max_num_seqs=4, max_num_batched_tokens=64,
                context_len=128)
    base.update(kw)
    return EngineConfig(model=model_dir, **base)


def test_dead_tp_worker_is_reported_not_waited_for(tiny_model_dir):
    eng = Engine(_cfg(tiny_model_dir, tp_size=2, nccl_port=29761))
    try:
        ex = eng._client.engine_core.executor
        eng.add_request([1, 2, 3], SamplingParams(max_tokens=50, ignore_eos=True))
        eng.step()
        victim = ex._procs[0]
        os.kill(victim.pid, signal.SIGKILL)        # the exact child this test's engine started
        victim.join(timeout=10)
        t0 = time.time()
        with pytest.raises(RuntimeError, match="worker process .* exited"):
            for _ in range(5):
                eng.step()
        assert time.time() - t0 < 30
    finally:
        ex._procs.clear()
        try:
            ex.worker.destroy_environment()
        except Exception:
            pass


def test_dead_dp_replica_fails_its_requests(tiny_model_dir):
    eng = Engine(_cfg(tiny_model_dir, dp_size=2, nccl_port=29771))
    try:
        client = eng._client
        for _ in range(4):
            eng.add_request([5, 6, 7, 8], SamplingParams(max_tokens=200, ignore_eos=True))
        eng.step()
        os.kill(client._procs[1].pid, signal.SIGKILL)
        client._procs[1].join(timeout=10)
        with pytest.raises(RuntimeError, match="DP replica 1 failed"):
            for _ in range(400):
                eng.step()
    finally:
        eng.destroy()


def test_corrupt_and_truncated_safetensors_are_rejected(tmp_path):
    d = tmp_path / "ckpt"
    d.mkdir()
    good = d / "model.safetensors"
    write_safetensors(str(good), {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4)})
    src = SafetensorsSource(str(d))
    assert torch.equal(src.read("a", 1, 2, 1, 2), torch.tensor([[5.0, 6.0], [9.0, 10.0]]))
    src.close()
    raw = good.read_bytes()
    (d / "model.safetensors").write_bytes(raw[:-8])                 # data cut short
    src = SafetensorsSource(str(d))
    with pytest.raises((ValueError, Exception)):
        src.read("a")
    src.close()
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 10) + b"{not json}")
    with pytest.raises(ValueError, match="corrupt safetensors header"):
        SafetensorsSource(str(d))
    (d / "model.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="exceeds file size"):
        SafetensorsSource(str(d))
    os.remove(d / "model.safetensors")
    with pytest.raises(FileNotFoundError):
        SafetensorsSource(str(d))


def test_config_validation(tmp_path, tiny_model_dir):
    with pytest.raises(FileNotFoundError):
        EngineConfig(model=str(tmp_path / "nope"))
    for bad in (dict(kvcache_block_size=8), dict(kvcache_block_size=24), dict(prefix_backend="lru"),
                dict(tp_size=0), dict(max_num_seqs=0), dict(load_format="pickle"), dict(device="tpu"),
                dict(pp_size=2, pp_layer_counts=[1, 2, 3]), dict(pp_size=2, pp_layer_counts=[5, 5])):
        with pytest.raises(ValueError):
            EngineConfig(model=tiny_model_dir, **bad)
    cfg = EngineConfig(model=tiny_model_dir, context_len=10 ** 9, tp_size=2, pp_size=2, dp_size=3)
    assert cfg.context_len == cfg.hf_config.max_position_embeddings
    assert (cfg.world_size, cfg.num_gpus, cfg.block_size) == (4, 12, 16)


def _ring_reader(path, world, rank, n, q):
    from xixi_vllm_b200.parallel.control_channel import _ShmRing
    ring = _ShmRing(path, world, rank, create=False)
    q.put(("attached", rank))
    try:
        got = [ring.read()[0] for _ in range(n)]
        q.put(("read", got))
    except RuntimeError as e:
        q.put(("error", str(e)))


def test_control_ring_notices_a_dead_reader_and_a_dead_writer(tmp_path):
    """Shared-memory control ring, host-side failure detection: a writer whose reader died stops with an
    error once the ring is full instead of waiting for acknowledgements forever; a reader whose writer
    died leaves its polling loop."""
    import multiprocessing as mp
    import os

    from xixi_vllm_b200.parallel.control_channel import _SLOTS, _ShmRing
    ctx = mp.get_context("spawn")
    # 1. reader reads two messages and exits; the writer fills the ring and must then raise
    path = str(tmp_path / "ring_a")
    ring = _ShmRing(path, 2, 0, create=True)
    q = ctx.Queue()
    p = ctx.Process(target=_ring_reader, args=(path, 2, 1, 2, q))
    p.start()
    assert q.get(timeout=60)[0] == "attached"
    ring.write(b"one")
    ring.write(b"two")
    assert q.get(timeout=60) == ("read", [b"one", b"two"])
    p.join(timeout=30)
    with pytest.raises(RuntimeError, match="is gone"):
        for i in range(_SLOTS + 2):
            ring.write(b"x%d" % i)
    ring.close()
    assert not os.path.exists(path)
    # 2. the writer side disappears (its pid in the header no longer exists): a waiting reader gives up
    path = str(tmp_path / "ring_b")
    ring = _ShmRing(path, 2, 0, create=True)
    dead = ctx.Process(target=int)          # a process that has exited: its pid is free
    dead.start()
    dead.join()
    import struct
    struct.pack_into("<Q", ring.map, 0, dead.pid)
    q = ctx.Queue()
    p = ctx.Process(target=_ring_reader, args=(path, 2, 1, 1, q))
    p.start()
    assert q.get(timeout=60)[0] == "attached"
    kind, msg = q.get(timeout=60)
    assert kind == "error" and "gone" in msg
    p.join(timeout=30)
    ring.close()
