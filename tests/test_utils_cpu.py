"""Framework utilities on CPU: precision plugin, debug hooks, safe tar extraction, env parsing, sharded checkpoint IO,
config version upgrade, sequence-length resolver, object-store URL handling."""
import io
import operator
import os
import tarfile

import pytest
import torch

from speech_b200.utils import misc


def test_half_precision_for_audio_keeps_waveforms_fp32():
    b = misc.HalfPrecisionForAudio("bf16-mixed").convert_input({"audio": torch.zeros(2, 8), "feats": torch.zeros(2, 3), "ids": torch.zeros(2, dtype=torch.long),
                                                                "nested": [torch.zeros(1)]})
    assert b["audio"].dtype == torch.float32 and b["feats"].dtype == torch.bfloat16 and b["ids"].dtype == torch.long
    assert b["nested"][0].dtype == torch.bfloat16


def test_debug_hooks_and_nvtx_noop():
    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU(), torch.nn.Linear(4, 2))
    lines = []
    hs = misc.register_debug_hooks(m, sink=lines.append)
    m(torch.randn(3, 4)).sum().backward()
    assert any(l.startswith("debug_info_forward/0") for l in lines) and any(l.startswith("debug_info_backward/2") for l in lines)
    for h in hs:
        h.remove()
    with misc.nvtx_range("x"):
        pass


def test_safe_extract_blocks_traversal(tmp_path):
    good = tmp_path / "good.tar"
    with tarfile.open(good, "w") as tf:
        data = b"hello"
        ti = tarfile.TarInfo("a/b.txt")
        ti.size = len(data)
        tf.addfile(ti, io.BytesIO(data))
    with tarfile.open(good) as tf:
        misc.safe_extract(tf, str(tmp_path / "out"))
    assert (tmp_path / "out" / "a" / "b.txt").read_bytes() == b"hello"
    bad = tmp_path / "bad.tar"
    with tarfile.open(bad, "w") as tf:
        ti = tarfile.TarInfo("../evil.txt")
        ti.size = 1
        tf.addfile(ti, io.BytesIO(b"x"))
    with tarfile.open(bad) as tf, pytest.raises(ValueError):
        misc.safe_extract(tf, str(tmp_path / "out2"))
    assert not (tmp_path / "evil.txt").exists()


def test_env_parsing_imports_versions_and_paths(monkeypatch):
    monkeypatch.setenv("SB_FLAG", "yes")
    assert misc.get_envbool("SB_FLAG") and not misc.get_envbool("SB_MISSING") and misc.get_envint("SB_MISSING", 3) == 3
    monkeypatch.setenv("SB_FLAG", "maybe")
    with pytest.raises(ValueError):
        misc.get_envbool("SB_FLAG")
    assert misc.safe_import("definitely_not_a_module")[1] is False and misc.safe_import("json")[1] is True
    ok, msg = misc.check_lib_version("torch", "1.0", operator.ge)
    assert ok and "satisfies" in msg
    assert misc.inject_model_parallel_rank("/x/y.ckpt", 1, 2) == "/x/mp_rank_01/y.ckpt"
    assert misc.inject_model_parallel_rank("/x/y.ckpt") == "/x/y.ckpt"
    assert misc.object_store_url("s3://bucket/key") == "s3" and misc.object_store_url("/local") is None
    with pytest.raises(FileNotFoundError):
        misc.maybe_download_from_cloud("https://example.invalid/", "m.nemo", cache_dir="/nonexistent-cache")


def test_config_upgrade_and_length_resolver():
    cfg = misc.maybe_update_config_version({"encoder": {"cls": "a.B", "params": {"x": 1, "inner": {"cls": "c.D", "params": {"y": 2}}}}})
    assert cfg.encoder["_target_"] == "a.B" and cfg.encoder.inner["_target_"] == "c.D" and cfg.encoder.inner.y == 2
    r = misc.SequenceLengthResolver({"inputs": [{"name": "audio", "type": "audio", "seq_length": "input"},
                                               {"name": "audio_len", "type": "lengths", "seq_length": "input"},
                                               {"name": "tokens", "type": "labels", "seq_length": "output", "vocab_size": 10}]})
    b = r(3, 1600, 7)
    assert b["audio"].shape == (3, 1600) and b["audio_len"].tolist() == [1600] * 3 and b["tokens"].shape == (3, 7)


def test_sharded_checkpoint_io_sync_and_async(tmp_path):
    io_ = misc.ShardedCheckpointIO(async_save=True)
    io_.save({"exp_avg": torch.arange(4.0), "step": 3}, str(tmp_path / "ck"), common={"global_step": 3})
    io_.wait()
    back = io_.load(str(tmp_path / "ck"))
    assert back["step"] == 3 and torch.equal(back["exp_avg"], torch.arange(4.0))
    assert len(io_.load_all(str(tmp_path / "ck"))) == 1
