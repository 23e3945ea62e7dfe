"""Checkpoint integrity / compatibility checks, typed state dicts, per-strategy collection, resharding strategies, factory."""
import json
import os

import pytest
import torch
import torch.nn as nn

from ml_framework_b200 import native_available
from ml_framework_b200.checkpoint import validation as V
from ml_framework_b200.checkpoint.distributed import (CheckpointCoordinator, CheckpointError, CheckpointLoader, CheckpointMetadata, LoadOptions,
                                                     manifest_path)
from ml_framework_b200.dist.process_group import run_fake_world

pytestmark = pytest.mark.skipif(not native_available(), reason="native library not built")


def _save_tp(tmp, world=2):
    torch.manual_seed(0)
    full = {"w": torch.randn(8, 6), "b": torch.randn(6), "col": torch.randn(4, 12)}
    dims = {"w": 0, "b": None, "col": 1}

    def worker(pg):
        local = {"w": full["w"].chunk(world, 0)[pg.rank], "b": full["b"], "col": full["col"].chunk(world, 1)[pg.rank]}
        tensors, info = V.DistributedStateCollector(pg.rank, world).collect("tp", local, shard_dims=dims)
        return CheckpointCoordinator(pg).coordinate_save(os.path.join(tmp, "ck"), tensors, info)
    metas = run_fake_world(world, worker)
    return full, metas[0], os.path.join(tmp, "ck")


def test_validator_passes_a_good_checkpoint_and_finds_damage(tmp_path):
    full, meta, prefix = _save_tp(str(tmp_path))
    rep = V.CheckpointValidator().validate(prefix)
    assert rep.is_valid and rep.errors() == []
    assert [t.Name for t in meta.Shards[1].Tensors] == ["w", "col"]              # replicated bias written by rank 0 only
    shard1 = os.path.join(str(tmp_path), meta.Shards[1].FilePath)
    raw = bytearray(open(shard1, "rb").read())
    raw[-3] ^= 0xFF
    open(shard1, "wb").write(raw)
    bad = V.CheckpointValidator().validate(prefix)
    assert not bad.is_valid and any(e.startswith("checksum:") for e in bad.errors()) and V.CheckpointValidator(quick=True).validate(prefix).is_valid
    open(shard1, "wb").write(raw[:-10])
    assert any("bytes on disk" in e for e in V.CheckpointValidator().validate(prefix).errors())
    os.remove(shard1)
    assert any("is missing" in e for e in V.SizeIntegrityChecker().check(prefix, meta).errors())
    assert V.ChecksumIntegrityChecker().check(prefix, meta).is_valid                  # missing files are the size check's finding
    assert V.CheckpointValidator().validate(os.path.join(str(tmp_path), "none")).errors()[0].startswith("manifest: no manifest")
    open(manifest_path(prefix), "w").write("{broken")
    assert "cannot be parsed" in V.CheckpointValidator().validate(prefix).errors()[0]


def test_version_and_schema_compatibility(tmp_path):
    _, meta, prefix = _save_tp(str(tmp_path))
    vc = V.VersionCompatibilityChecker("1.2.0")
    meta.Version = "1.1.0"
    assert vc.check(meta).issues == []
    meta.Version = "1.3.0"
    r = vc.check(meta)
    assert r.is_valid and "newer than this reader" in r.warnings()[0]
    meta.Version = "2.0.0"
    assert not vc.check(meta).is_valid
    meta.Version = "one"
    assert "not a version" in vc.check(meta).errors()[0]
    meta.Version = "1.0.0"
    sc = V.SchemaCompatibilityChecker()
    assert sc.check(meta).is_valid
    t = meta.Shards[0].Tensors[0]
    t.Size += 4
    assert any("!= " in e for e in sc.check(meta).errors())
    t.Size -= 4
    t.DataType = "float19"
    assert any("unknown data type" in e for e in sc.check(meta).errors())
    t.DataType = "float32"
    meta.Shards[1].Tensors[0].ShardIndex = 0
    assert any("slice indices" in e for e in sc.check(meta).errors())
    meta.Shards[1].Tensors[0].ShardIndex = 1
    meta.Shards[1].Tensors[0].GlobalShape = [99, 6]
    assert any("disagree" in e for e in sc.check(meta).errors())
    meta.Shards[1].Tensors[0].GlobalShape = [8, 6]
    meta.Shards[1].Tensors[0].Shape = [2, 6]
    meta.Shards[1].Tensors[0].Size = 48
    assert any("slices cover 6 of 8" in e for e in sc.check(meta).errors())
    meta.Shards.pop()
    assert any("expected 2 shards" in e for e in sc.check(meta).errors())


def test_simple_and_parallel_resharding_agree(tmp_path):
    full, meta, prefix = _save_tp(str(tmp_path), world=4)
    for target in (1, 2, 3):
        for r in range(target):
            a = V.resharding_strategy("parallel").load(meta, prefix, target, r)
            b = V.resharding_strategy("simple").load(meta, prefix, target, r)
            assert set(a) == set(b) == {"w", "b", "col"}
            for k in a:
                assert torch.equal(a[k], b[k])
            per = -(-8 // target)
            assert torch.equal(a["w"], full["w"][r * per:(r + 1) * per]) and torch.equal(a["b"], full["b"])
    res = CheckpointLoader().coordinate_load(prefix, LoadOptions(resharding_strategy="simple"))
    assert res.was_resharded and torch.equal(res.tensors["col"], full["col"])
    with pytest.raises(KeyError):
        V.resharding_strategy("magic")


def test_typed_state_dicts_and_compatibility_checker():
    m = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
    sd = V.ModelStateDict.from_module(m)
    assert sd.kind == "model" and sd.total_bytes() == 4 * (12 + 3 + 6 + 2) and len(sd.fingerprint()) == 16
    assert V.ModelStateDict.from_module(nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))).fingerprint() == sd.fingerprint()
    assert sd.with_prefix("model.").strip_prefix("model.").keys() == sd.keys() and sd.with_prefix("m.").fingerprint() != sd.fingerprint()
    opt = torch.optim.Adam(m.parameters(), lr=0.1)
    m(torch.randn(5, 4)).sum().backward()
    opt.step()
    osd = V.OptimizerStateDict.from_optimizer(opt)
    assert "state.0.exp_avg" in osd and osd.extras["param_groups"][0]["lr"] == 0.1 and osd.kind == "optimizer"
    back = osd.to_optimizer_state()
    opt2 = torch.optim.Adam(m.parameters(), lr=0.5)
    opt2.load_state_dict(back)
    assert torch.equal(opt2.state_dict()["state"][0]["exp_avg"], opt.state_dict()["state"][0]["exp_avg"]) and opt2.param_groups[0]["lr"] == 0.1
    chk = V.StateCompatibilityChecker()
    ck = {k: v.clone() for k, v in sd.items()}
    assert chk.check(ck, m.state_dict()).describe() == "compatible"
    ck["extra"] = torch.zeros(1)
    del ck["2.bias"]
    ck["0.weight"] = ck["0.weight"].half()
    c = chk.check(ck, m.state_dict())
    assert c.missing == ["2.bias"] and c.unexpected == ["extra"] and c.dtype_mismatches[0][0] == "0.weight" and not c.is_compatible() and c.is_compatible(strict=False)
    with pytest.raises(CheckpointError, match="missing"):
        chk.load_checked(m, ck)
    before = m[2].bias.clone()
    chk.load_checked(m, ck, strict=False)
    assert torch.equal(m[2].bias, before) and m[0].weight.dtype == torch.float32
    ck["2.weight"] = torch.zeros(5, 5)
    assert not chk.check(ck, m.state_dict()).is_compatible(strict=False) and "checkpoint (5, 5), target (2, 3)" in chk.check(ck, m.state_dict()).describe()


def test_collectors_for_ddp_and_fsdp_and_the_factory(tmp_path):
    st = {"a": torch.arange(4.0)}
    assert V.DDPCheckpointHelper.collect_full_state(st, 0)[0].keys() == st.keys() and V.DDPCheckpointHelper.collect_full_state(st, 1) == ({}, {})
    flat = torch.arange(10.0)
    loc, info = V.DistributedStateCollector(1, 4).collect("fsdp", {"flat": flat[3:6]}, global_numel={"flat": 10})
    assert info["flat"] == {"GlobalShape": [10], "ShardDim": 0, "ShardIndex": 1, "ShardCount": 4} and torch.equal(loc["flat"], flat[3:6])
    dst = {"flat": torch.zeros(4), "other": torch.zeros(2)}
    assert V.FSDPCheckpointHelper.load_local_shard({"flat": torch.tensor([1.0, 2.0, 3.0])}, dst) == ["other"] and dst["flat"].tolist() == [1.0, 2.0, 3.0, 0.0]
    with pytest.raises(KeyError):
        V.DistributedStateCollector(0, 1).collect("zero9", {})
    o = V.CheckpointOptions(directory=str(tmp_path / "ck"), max_to_keep=2, compression=V.CheckpointCompressionLevel.NONE)
    assert o.save_options().format == "multishard" and o.load_options(strict=False).resharding_strategy == "parallel"
    ck = V.DistributedCheckpointFactory.create_validated(o)
    for i in range(3):
        ck.save(f"t{i}", {"w": torch.full((3,), float(i))}, step=i)
    assert ck.list_checkpoints() == ["t1", "t2"] and ck.load("t2").tensors["model.w"].tolist() == [2.0, 2.0, 2.0]
    with pytest.raises(ValueError):
        V.DistributedCheckpointFactory.create(V.CheckpointOptions(max_to_keep=-1))
    with pytest.raises(KeyError):
        V.DistributedCheckpointFactory.create(V.CheckpointOptions(resharding_strategy="none"))
    assert V.CheckpointFormat("singlefile") == V.CheckpointFormat.SINGLE_FILE
