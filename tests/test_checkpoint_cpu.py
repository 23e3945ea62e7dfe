"""Multi-shard checkpoint format: round trip, corruption detection (magic, rank, checksum, tensor
count), resharding across world sizes, async and incremental managers, retry / circuit breaker."""
import os
import struct
import time

import pytest
import torch

from ml_framework_b200.checkpoint.distributed import (AsyncCheckpointManager, CheckpointCorruptError, CheckpointError,
                                                      CheckpointLoader, CheckpointMetadata, CircuitBreaker,
                                                      DistributedCheckpoint, FaultToleranceHandler, IncrementalCheckpointManager,
                                                      LoadOptions, MultiShardCheckpointFormat, RetryPolicy, SaveOptions,
                                                      ShardFileVerifier, SingleFileCheckpointFormat, manifest_path, shard_path)
from ml_framework_b200.dist.process_group import run_fake_world


def _state(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"w": torch.randn(6, 4, generator=g), "b": torch.randn(4, generator=g).to(torch.bfloat16),
            "step": torch.tensor([7], dtype=torch.int64)}


def test_shard_file_layout_and_round_trip(tmp_path):
    p = str(tmp_path / "ck_shard_0.shard")
    st = _state()
    meta = MultiShardCheckpointFormat.write_shard(p, 0, st)
    raw = open(p, "rb").read()
    magic, rank, clen = struct.unpack("<iii", raw[:12])
    assert magic == 0x53484152 and rank == 0 and clen == 64
    assert raw[12:76].decode() == meta.Checksum
    tcount, dlen = struct.unpack("<ii", raw[76:84])
    assert tcount == 3 and dlen == sum(t.Size for t in meta.Tensors) and len(raw) == 84 + dlen == meta.FileSize
    back = MultiShardCheckpointFormat.read_shard(p, meta)
    for k in st:
        assert torch.equal(back[k], st[k]) and back[k].dtype == st[k].dtype


def test_corruption_is_detected(tmp_path):
    p = str(tmp_path / "x_shard_1.shard")
    meta = MultiShardCheckpointFormat.write_shard(p, 1, _state())
    raw = bytearray(open(p, "rb").read())

    def write(b):
        open(p, "wb").write(b)
    bad = bytearray(raw); bad[0] ^= 0xFF; write(bad)
    with pytest.raises(CheckpointCorruptError, match="magic"):
        MultiShardCheckpointFormat.read_shard(p, meta)
    write(raw)
    meta.Rank = 0
    with pytest.raises(CheckpointCorruptError, match="rank"):
        MultiShardCheckpointFormat.read_shard(p, meta)
    meta.Rank = 1
    bad = bytearray(raw); bad[-1] ^= 0x01; write(bad)
    with pytest.raises(CheckpointCorruptError, match="checksum"):
        MultiShardCheckpointFormat.read_shard(p, meta)
    write(raw)
    meta.Tensors.pop()
    with pytest.raises(CheckpointCorruptError, match="count"):
        MultiShardCheckpointFormat.read_shard(p, meta)
    write(raw[:40])
    with pytest.raises(CheckpointCorruptError):
        MultiShardCheckpointFormat.read_header(p)


def test_save_load_same_world_and_resharded(tmp_path):
    full = torch.arange(8 * 3, dtype=torch.float32).reshape(8, 3)
    rep = torch.tensor([1.0, 2.0])

    def save(pg):
        W, r = pg.world_size, pg.rank
        ck = DistributedCheckpoint(str(tmp_path), pg)
        ck.save("t1", {"w": full.chunk(W, 0)[r].clone(), "rep": rep},
                slice_info={"w": {"GlobalShape": [8, 3], "ShardDim": 0, "ShardIndex": r, "ShardCount": W}},
                step=5, strategy="fsdp")
        return ck.load("t1").tensors["model.w"]
    outs = run_fake_world(4, save)
    assert torch.equal(torch.cat(outs), full)
    meta = CheckpointLoader().load_metadata(str(tmp_path / "t1"))
    assert meta.WorldSize == 4 and meta.Training.Step == 5 and meta.Format == "multishard" and len(meta.Shards) == 4
    assert os.path.exists(shard_path(str(tmp_path / "t1"), 3)) and os.path.exists(manifest_path(str(tmp_path / "t1")))
    ok, errs = ShardFileVerifier.verify_checkpoint(str(tmp_path / "t1"))
    assert ok, errs

    def load2(pg):
        res = DistributedCheckpoint(str(tmp_path), pg).load("t1")
        assert res.was_resharded and res.source_world_size == 4 and res.target_world_size == 2
        assert torch.equal(res.tensors["model.rep"], rep)
        return res.tensors["model.w"]
    outs = run_fake_world(2, load2)
    assert torch.equal(torch.cat(outs), full) and outs[0].shape == (4, 3)
    one = DistributedCheckpoint(str(tmp_path)).load("t1")
    assert torch.equal(one.tensors["model.w"], full)
    # three target ranks: uneven split ceil(8/3) = 3, 3, 2
    outs = run_fake_world(3, lambda pg: DistributedCheckpoint(str(tmp_path), pg).load("t1").tensors["model.w"])
    assert [o.shape[0] for o in outs] == [3, 3, 2] and torch.equal(torch.cat(outs), full)


def test_single_file_async_incremental_and_retention(tmp_path):
    st = _state(1)
    ck = DistributedCheckpoint(str(tmp_path), max_to_keep=2)
    ck.save("s", st, options=SaveOptions(format="singlefile"))
    got = ck.load("s").tensors
    assert torch.equal(got["model.w"], st["w"])
    mgr = AsyncCheckpointManager(ck)
    for i in range(3):
        mgr.queue_save(f"a{i}", {"w": st["w"] + i})
    res = mgr.wait_for_completion()
    mgr.shutdown()
    assert set(res) == {"a0", "a1", "a2"} and ck.list_checkpoints() == ["a1", "a2"]
    assert torch.equal(ck.load("a2", LoadOptions(load_optimizer=False)).tensors["model.w"], st["w"] + 2)
    inc = IncrementalCheckpointManager(str(tmp_path / "inc"))
    inc.save_baseline("b", st)
    st2 = dict(st); st2["b"] = st["b"] + 1
    assert inc.save_incremental("d1", st2) == ["b"]
    assert torch.equal(inc.load()["b"], st2["b"]) and torch.equal(inc.load()["w"], st["w"])


def test_retry_and_circuit_breaker():
    calls, sleeps = [], []

    def flaky():
        calls.append(1)
        if len(calls) < 3:
            raise IOError("disk")
        return "ok"
    h = FaultToleranceHandler(RetryPolicy(max_retries=3, initial_delay_s=1.0), sleep=sleeps.append)
    assert h.execute_with_retry(flaky) == "ok" and sleeps == [1.0, 2.0]
    now = [0.0]
    br = CircuitBreaker(threshold=2, reset_s=10.0, clock=lambda: now[0])
    h = FaultToleranceHandler(RetryPolicy(max_retries=5, initial_delay_s=0.0), br, sleep=lambda s: None)
    with pytest.raises(CheckpointError, match="circuit breaker"):
        h.execute_with_retry(lambda: (_ for _ in ()).throw(IOError("x")))
    assert br.state == "open" and h.attempts == 2
    now[0] = 11.0
    assert br.state == "half_open" and br.allow()
    with pytest.raises(CheckpointError, match="timed out"):
        import time
        FaultToleranceHandler().execute_with_timeout(lambda: time.sleep(1.0), 0.05)
    assert RetryPolicy().delay(10) == 30.0


def test_storage_backend_rollback_manager_cancel_and_timeouts(tmp_path):
    from ml_framework_b200.checkpoint.distributed import (CheckpointCorruptError, CheckpointRollbackManager, LocalFileSystemStorage,
                                                          StorageFactory, manifest_path, shard_path)
    st = StorageFactory.create("local", root=str(tmp_path / "store"))
    assert isinstance(st, LocalFileSystemStorage) and st.list() == []
    st.write("a/b.bin", b"hello")
    st.write("top.bin", b"12345678")
    assert st.exists("a/b.bin") and st.read("a/b.bin") == b"hello" and st.get_metadata("top.bin")["size"] == 8
    assert st.list("top") == ["top.bin"] and st.path("/abs/x") == "/abs/x"
    st.delete("top.bin")
    st.delete("top.bin")                                            # deleting what is gone is not an error
    assert not st.exists("top.bin")
    with pytest.raises(ValueError):
        StorageFactory.create("s3")
    ck = DistributedCheckpoint(str(tmp_path / "ck"), max_to_keep=0)
    s0 = _state(2)
    ck.save_model_only("good", s0, step=7)
    assert set(ck.load("good").tensors) == {"model." + k for k in s0} and ck.load("good").metadata.Training.Step == 7
    rb = CheckpointRollbackManager(ck)
    with pytest.raises(CheckpointError):
        rb.rollback()                                               # nothing verified yet
    rb.mark_good("good")
    ck.save("bad", {"w": s0["w"] * 2})
    with open(shard_path(ck._prefix("bad"), 0), "r+b") as f:         # damage the newer checkpoint
        f.seek(200)
        f.write(b"\\xff" * 16)
    with pytest.raises(CheckpointCorruptError):
        rb.mark_good("bad")
    back = rb.rollback()
    assert rb.last_good == "good" and torch.equal(back.tensors["model.w"], s0["w"])
    ck.save("one", s0, options=SaveOptions(format="singlefile"))
    assert os.path.exists(ck._prefix("one") + ".ckpt")
    ck.delete("one")
    ck.delete("bad")
    assert not os.path.exists(ck._prefix("one") + ".ckpt") and not os.path.exists(manifest_path(ck._prefix("bad")))
    assert ck.list_checkpoints() == ["good"]
    mgr = AsyncCheckpointManager(ck, max_pending=4)
    mgr.cancel_checkpoint("skip-me")
    mgr.queue_save("keep-me", s0)
    mgr.queue_save("skip-me", s0)
    mgr.wait_for_completion()
    mgr.shutdown()
    assert "keep-me" in ck.list_checkpoints() and "skip-me" not in ck.list_checkpoints()
    h = FaultToleranceHandler(RetryPolicy(max_retries=0), sleep=lambda s: None)
    import time as _t
    with pytest.raises(CheckpointError, match="timed out"):
        h.execute_with_timeout(lambda: _t.sleep(1.0), 0.05)
    assert h.execute_with_timeout(lambda a, b=1: a + b, 1.0, 2, b=3) == 5
    with pytest.raises(KeyError):
        h.execute_with_timeout(lambda: {}["x"], 1.0)


def test_async_checkpoint_tasks_are_tracked(tmp_path):
    import threading

    from ml_framework_b200.checkpoint.distributed import (CheckpointQueueFullError, CheckpointTaskStatus, CheckpointTaskType)
    gate = threading.Event()

    class Slow(DistributedCheckpoint):
        def save(self, tag, *a, **k):
            if tag == "first":
                gate.wait(10)
            if tag == "bad":
                raise IOError("disk full")
            return super().save(tag, *a, **k)

    st = _state(2)
    mgr = AsyncCheckpointManager(Slow(str(tmp_path)), max_pending=2)
    mgr.queue_save("first", st, {"m": torch.zeros(3)})
    for _ in range(200):
        if mgr.get_task_status("first") is CheckpointTaskStatus.RUNNING:
            break
        time.sleep(0.01)
    mgr.queue_save("second", st)
    mgr.queue_save("bad", st)
    with pytest.raises(CheckpointQueueFullError):
        mgr.queue_save("fourth", st, block=False)
    with pytest.raises(CheckpointError, match="still in flight"):
        mgr.queue_save("second", st)
    assert mgr.get_task_status("first") is CheckpointTaskStatus.RUNNING and mgr.get_task_status("second") is CheckpointTaskStatus.QUEUED
    assert mgr.get_task_info("first").type is CheckpointTaskType.FULL and mgr.get_task_info("second").type is CheckpointTaskType.MODEL_ONLY
    assert {t.id for t in mgr.get_active_tasks()} == {"first", "second", "bad"} and mgr.active_task_count == 3 and mgr.queue_size == 2
    assert mgr.cancel_checkpoint("second") and not mgr.cancel_checkpoint("first") and mgr.get_task_status("nope") is None
    gate.set()
    r1, r2, r3 = mgr.wait_for("first"), mgr.wait_for("second"), mgr.wait_for("bad")
    assert r1.success and r1.bytes_snapshotted > 0 and r1.duration_s >= 0
    assert not r2.success and mgr.get_task_status("second") is CheckpointTaskStatus.CANCELLED
    assert not r3.success and isinstance(r3.error, IOError) and mgr.get_task_status("bad") is CheckpointTaskStatus.FAILED
    info = mgr.get_task_info("first")
    assert info.status is CheckpointTaskStatus.COMPLETED and info.duration_s is not None and mgr.active_task_count == 0
    with pytest.raises(CheckpointError, match="async saves failed"):
        mgr.wait_for_completion()
    with pytest.raises(KeyError):
        mgr.wait_for("nope")
    mgr.shutdown()
