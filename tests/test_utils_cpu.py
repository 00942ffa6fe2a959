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


def test_callback_group_object_store_io_and_hf_directory(tmp_path):
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.utils.callbacks_extra import (CallbackGroup, EventRecorder, HuggingFaceFileIO, NsightProfiling, ObjectStoreCheckpointIO,
                                                   StaticBufferLoader, hook_class_init_with_callbacks)

    group = CallbackGroup.get_instance()
    group.clear()
    rec = EventRecorder(clock=iter(range(100)).__next__)
    group.register(rec)
    assert CallbackGroup.get_instance() is group

    class Thing:
        def __init__(self, v):
            self.v = v

    hook_class_init_with_callbacks(Thing, "on_model_init_start", "on_model_init_end")
    assert Thing(3).v == 3
    group.on_save_checkpoint_start(iteration=1)
    group.some_event_nobody_handles()
    assert [e for e, _ in rec.events] == ["on_model_init_start", "on_model_init_end", "on_save_checkpoint_start"]
    group.clear()

    class FakeS3:
        def __init__(self):
            self.store = {}

        def upload_file(self, local, bucket, key):
            self.store[(bucket, key)] = open(local, "rb").read()

        def download_file(self, bucket, key, local):
            open(local, "wb").write(self.store[(bucket, key)])

        def delete_object(self, Bucket, Key):
            del self.store[(Bucket, Key)]

    s3 = FakeS3()
    io = ObjectStoreCheckpointIO(client=s3, staging_dir=str(tmp_path / "stage"), async_checkpointing=True)
    io.save_checkpoint({"w": torch.arange(4)}, "s3://bucket/run/step=4.ckpt")
    io.wait()
    assert ("bucket", "run/step=4.ckpt") in s3.store and not os.listdir(tmp_path / "stage")
    assert torch.equal(io.load_checkpoint("s3://bucket/run/step=4.ckpt")["w"], torch.arange(4))
    io.remove_checkpoint("s3://bucket/run/step=4.ckpt")
    assert not s3.store
    io.save_checkpoint({"w": torch.ones(2)}, str(tmp_path / "local" / "a.ckpt"))
    assert torch.equal(io.load_checkpoint(str(tmp_path / "local" / "a.ckpt"))["w"], torch.ones(2))
    with pytest.raises(ImportError):
        ObjectStoreCheckpointIO(staging_dir=str(tmp_path / "stage")).load_checkpoint("s3://b/k")

    from speech_b200.core.instantiate import allow_prefix

    allow_prefix("test_utils_cpu.")
    global _TinyHF

    class _TinyHF(torch.nn.Module, HuggingFaceFileIO):
        def __init__(self, cfg):
            super().__init__()
            self.cfg = cfg
            self.lin = torch.nn.Linear(cfg.d, cfg.d)

    m = _TinyHF(OmegaConf.create({"d": 3}))
    m.save_pretrained(str(tmp_path / "hf"))
    again = _TinyHF.from_pretrained(str(tmp_path / "hf"))
    assert torch.equal(again.lin.weight, m.lin.weight)
    with pytest.raises((FileNotFoundError, Exception)):
        _TinyHF.from_pretrained(str(tmp_path / "missing"))
    loader = StaticBufferLoader(torch.device("cpu"))
    a = loader.load((torch.ones(2, 3), {"k": torch.zeros(4)}))
    b = loader.load((torch.full((2, 3), 5.0), {"k": torch.ones(4)}))
    assert a[0] is b[0] and float(b[0][0, 0]) == 5.0 and len(loader.buffers) == 1
    with pytest.raises(ValueError):
        NsightProfiling(5, 2)


def test_extra_tokenizers_and_chat_template():
    from speech_b200.tokenizers import ByteLevelTokenizer
    from speech_b200.tokenizers.extra import (ChatTemplateMixin, ChineseCharsTokenizer, EnJaProcessor, MosesProcessor, NullTokenizer, RegExTokenizer,
                                              TiktokenTokenizer, WordTokenizer)

    w = WordTokenizer(vocab=["hello", "world"], bos_token="<s>", eos_token="</s>")
    assert w.text_to_ids("hello there world") == [4, w.unk_id, 5] and w.ids_to_text([4, 5]) == "hello world" and w.vocab_size == 6
    r = RegExTokenizer()
    r.build_vocab_from_text(["CC(=O)Cl", "[NH4+]Br"])
    ids = r.text_to_ids("CC(=O)Cl")
    assert r.ids_to_text(ids) == "CC(=O)Cl" and r.text_to_tokens("[NH4+]Br") == ["[NH4+]", "Br"]
    n = NullTokenizer(100)
    assert n.text_to_ids("3 14 15") == [3, 14, 15] and n.ids_to_text([9, 2]) == "9 2" and n.vocab_size == 100
    c = ChineseCharsTokenizer(vocab=list("你好世界") + ["ok"])
    toks = c.text_to_tokens("你好 ok 世界")
    assert toks == ["你", "好", "ok", "世", "界"] and c.tokens_to_text(toks) == "你好ok世界" and c.tokens_to_text(["ok", "go", "你"]) == "ok go你"
    mp = MosesProcessor("en")
    t = mp.tokenize("Hello, world! It's fine.")
    assert t == "Hello , world ! It 's fine ." and mp.detokenize(t.split()) == "Hello, world! It's fine."
    assert EnJaProcessor("ja").detokenize(EnJaProcessor("ja").tokenize("こんにちは").split()) == "こんにちは"
    try:
        import tiktoken  # noqa: F401
        have = True
    except ImportError:
        have = False
    if not have:
        with pytest.raises(ImportError):
            TiktokenTokenizer("missing.json")

    class Tok(ByteLevelTokenizer, ChatTemplateMixin):
        pass

    tk = Tok()
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]
    s = tk.apply_chat_template(msgs, add_generation_prompt=True)
    assert s == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\nyo<|im_end|>\n<|im_start|>assistant\n"
    enc = tk.apply_chat_template(msgs, tokenize=True)
    assert len(enc["input_ids"]) == len(enc["assistant_mask"]) and 0 < sum(enc["assistant_mask"]) < len(enc["input_ids"])
    assert tk.apply_chat_template(msgs, template="llama3").startswith("<|begin_of_text|><|start_header_id|>user")


def test_asr_evaluator_explorer_report_and_rir_generator(tmp_path):
    import json

    import numpy as np

    from speech_b200.data.rir_generator import RIRCorpusGenerator, image_source_rir, measure_rt60, sabine_reflection
    from speech_b200.utils.asr_evaluator import ASREvaluator, align_words, write_explorer_report
    from speech_b200.utils.metrics import word_error_rate_detail

    wer, n, ins, dele, sub = word_error_rate_detail(["a x c d e"], ["a b c d"])
    assert n == 4 and abs(wer - 0.5) < 1e-9 and abs(ins - 0.25) < 1e-9 and dele == 0 and abs(sub - 0.25) < 1e-9
    assert [op for op, _, _ in align_words("a b c d".split(), "a x c d e".split())] == ["ok", "sub", "ok", "ok", "ins"]
    man = tmp_path / "m.json"
    rows = [{"audio_filepath": f"/x/{i}.wav", "duration": 1.0 + 3 * i, "text": t, "gender": g}
            for i, (t, g) in enumerate([("hello world", "f"), ("good morning all", "m"), ("one two three four", "f")])]
    man.write_text("\n".join(json.dumps(r) for r in rows))
    fake = {"/x/0.wav": "hello world", "/x/1.wav": "good morning", "/x/2.wav": "one too three four"}
    ev = ASREvaluator(transcribe_fn=lambda paths: [fake[p] for p in paths])
    res = ev.run(str(man), str(tmp_path / "out"), metadata_keys=["gender"], duration_buckets=[3.0, 6.0])
    assert abs(res["wer"] - 2 / 9) < 1e-9 and abs(res["del_rate"] - 1 / 9) < 1e-9 and abs(res["sub_rate"] - 1 / 9) < 1e-9
    assert res["breakdown"]["gender"]["m"]["wer"] == pytest.approx(1 / 3) and res["breakdown"]["gender"]["f"]["utterances"] == 2
    assert set(res["breakdown"]["duration"]) == {"<3s", "3-6s", ">=6s"}
    preds = [json.loads(l) for l in (tmp_path / "out" / "predictions.json").read_text().splitlines()]
    assert preds[1]["pred_text"] == "good morning" and preds[1]["wer"] == pytest.approx(1 / 3)
    stats = write_explorer_report(preds, str(tmp_path / "report.html"))
    page = (tmp_path / "report.html").read_text()
    assert stats["utterances"] == 3 and ("sub", "two", "too", 1) in stats["top_errors"] and "two→too" in page and "<svg" in page
    # image-source room response: direct path first, at distance / c, and a decay close to the requested RT60
    room, src, mic = [6.0, 5.0, 3.0], [2.0, 2.5, 1.5], [4.0, 2.5, 1.5]
    h = image_source_rir(room, src, mic, rt60=0.4, sample_rate=16000, max_order=17)
    first = int(np.argmax(np.abs(h) > 0.5 * np.abs(h).max()))
    assert abs(first - 2.0 / 343.0 * 16000) <= 2
    assert 0 < sabine_reflection(room, 0.4) < 1 and sabine_reflection(room, 0.8) > sabine_reflection(room, 0.2)
    rt = measure_rt60(h, 16000, decay_db=20)
    assert 0.2 < rt < 0.8, rt
    with pytest.raises(ValueError):
        image_source_rir(room, [7.0, 1, 1], mic, 0.3)
    gen = RIRCorpusGenerator(num_mics=2, max_order=4, seed=1)
    path = gen.generate(str(tmp_path / "rirs"), 2)
    recs = [json.loads(l) for l in open(path)]
    assert len(recs) == 2 and len(recs[0]["mic_positions"]) == 2 and (tmp_path / "rirs" / "rir_00001.wav").exists()


def test_fp8_post_training_quantisation_calibrate_replace_report_roundtrip(tmp_path):
    import torch

    from speech_b200.utils.quantization import (QuantLinear, calibrate, load_quantized, quantization_report, quantize_model, save_quantized,
                                                to_e4m3)

    # e4m3 grid: exact values stay, 3 mantissa bits otherwise, saturation at 448
    x = torch.tensor([0.0, 1.0, 1.0625, 1.125, 3.3, 447.0, 1000.0, -0.3])
    q = to_e4m3(x)
    assert q.tolist()[:2] == [0.0, 1.0] and float(q[3]) == 1.125 and float(q[6]) == 448.0 and abs(float(q[4]) - 3.25) < 1e-6
    assert float((q[2] - 1.0).abs()) in (0.0, 0.125)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 16))
    batches = [(torch.randn(8, 32),) for _ in range(6)]
    amax = calibrate(net, batches, percentile=100.0)
    assert set(amax) == {"0", "2"} and amax["0"] > 2.0 and amax["2"] > 0
    only = calibrate(net, batches, skip=[r"^2$"])
    assert set(only) == {"0"}
    rep = quantization_report(net, amax)
    assert len(rep) == 2 and all(r["weight_sqnr_db"] > 25 for r in rep)          # about 6 dB per mantissa bit + the per-channel scale
    ref = net(batches[0][0])
    assert quantize_model(net, amax) == ["0", "2"] and isinstance(net[0], QuantLinear)
    out = net(batches[0][0])
    rel = float((out - ref).norm() / ref.norm())
    assert 0 < rel < 0.08, rel
    save_quantized(net, str(tmp_path / "q.pt"))
    fresh = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 16))
    load_quantized(fresh, str(tmp_path / "q.pt"))
    assert torch.equal(fresh(batches[0][0]), out)


def test_sharded_checkpoint_io_precision_timing_launcher_telemetry_punctuation(tmp_path):
    import sys

    import torch

    from speech_b200.utils.extras import (DeltaTimingCallback, DistributedCheckpointIO, FlashPrecision, ProcessLauncher, TelemetryCallback,
                                          punctuation_error_rate)

    # two "ranks" write one checkpoint: replicated tensors are spread over the ranks, the sharded one is stored piecewise
    full = {"a.weight": torch.randn(4, 3), "b.bias": torch.randn(5), "emb": torch.arange(12.0).view(6, 2)}
    path = str(tmp_path / "ckpt")
    ios = [DistributedCheckpointIO(rank=r, world_size=2, async_save=True) for r in range(2)]
    for r, io in enumerate(ios):
        st = dict(full, emb=full["emb"][3 * r: 3 * r + 3])
        io.save_checkpoint(st, path, sharded={"emb": 0}, extra={"step": 7})
    assert not DistributedCheckpointIO.is_complete(path)               # the index appears only after the writes are joined
    for io in reversed(ios):
        io.finalize()
    assert DistributedCheckpointIO.is_complete(path)
    got, extra = DistributedCheckpointIO.load_checkpoint(path)
    assert extra == {"step": 7} and all(torch.equal(got[k], full[k]) for k in full)
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4))
    net[1].register_parameter("norm_scale", torch.nn.Parameter(torch.ones(4)))
    FlashPrecision().convert_module(net)
    assert net[0].weight.dtype == torch.bfloat16 and net[1].norm_scale.dtype == torch.float32
    b = FlashPrecision().convert_input({"audio_signal": torch.zeros(2, 8), "features": torch.zeros(2, 8), "tokens": torch.zeros(2, 3, dtype=torch.long)})
    assert b["audio_signal"].dtype == torch.float32 and b["features"].dtype == torch.bfloat16 and b["tokens"].dtype == torch.long
    t = [0.0]

    class Tr:
        callback_metrics = {}

    cb = DeltaTimingCallback(clock=lambda: t[0])
    for dt in (1.0, 2.5):
        cb.on_train_batch_end(Tr, None, None, None, 0)
        t[0] += dt
    cb.on_train_batch_end(Tr, None, None, None, 0)
    assert Tr.callback_metrics["train_step_timing in s"] == 2.5
    tel = TelemetryCallback(path=str(tmp_path / "tel.jsonl"), clock=lambda: t[0])
    tel.on_model_init_start()
    t[0] += 3.0
    tel.on_model_init_end(params=10)
    assert tel.durations() == {"model_init": 3.0} and len(open(tmp_path / "tel.jsonl").read().splitlines()) == 2
    jobs = ProcessLauncher.expand_sweep({"lr": [1, 2], "bs": [8]})
    assert jobs == [["lr=1", "bs=8"], ["lr=2", "bs=8"]]
    code = "import sys, os; print(sys.argv[1:], os.environ.get('CUDA_VISIBLE_DEVICES')); sys.exit(3 if 'lr=2' in sys.argv else 0)"
    res = ProcessLauncher([sys.executable, "-c", code], gpu_ids=[5, 6], log_dir=str(tmp_path / "mr")).launch(jobs)
    assert [r[1] for r in res] == [0, 3] and "lr=1" in open(res[0][2]).read() and open(res[0][2]).read().strip()[-1] in "56"
    per = punctuation_error_rate(["hello, world how are you."], ["hello world, how are you?"])
    assert per[","]["insertions"] == 1 and per[","]["deletions"] == 1 and per["?"]["substitutions"] == 1 and per["overall"]["correct"] == 0
    assert punctuation_error_rate(["yes, it is."], ["yes, it is."])["overall"]["per"] == 0.0


def test_multirun_sweeps_and_model_utilities(tmp_path):
    import sys
    from speech_b200.core.config import OmegaConf, expand_multirun_overrides, hydra_runner
    from speech_b200.utils import misc

    assert expand_multirun_overrides(["lr=1e-3,1e-4", "size=small", "aug=[a,b],[c]"]) == [
        ["lr=1e-3", "size=small", "aug=[a,b]"], ["lr=1e-3", "size=small", "aug=[c]"],
        ["lr=1e-4", "size=small", "aug=[a,b]"], ["lr=1e-4", "size=small", "aug=[c]"]]
    (tmp_path / "c.yaml").write_text("lr: 0.1\nsize: tiny\nnested: {k: 1}\n")

    @hydra_runner(config_path=str(tmp_path), config_name="c")
    def main(cfg):
        return (cfg.lr, cfg.size, cfg.nested.k)

    assert main(argv=["lr=0.5"]) == (0.5, "tiny", 1)
    assert main(argv=["-m", "lr=0.5,0.25", "nested.k=7,8"]) == [(0.5, "tiny", 7), (0.5, "tiny", 8), (0.25, "tiny", 7), (0.25, "tiny", 8)]
    # child-process launcher: the same script is started once per job
    script = tmp_path / "job.py"
    script.write_text(
        "import sys\nsys.path.insert(0, %r)\nfrom speech_b200.core.config import hydra_runner\n"
        "@hydra_runner(config_path=%r, config_name='c')\ndef main(cfg):\n    print('JOB', cfg.lr, cfg.size)\n"
        "if __name__ == '__main__':\n    r = main()\n    print('RESULTS', r)\n" % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), str(tmp_path)))
    import subprocess
    out = subprocess.run([sys.executable, str(script), "-m", "lr=1,2", "size=a", "hydra.launcher.n_jobs=2", f"hydra.launcher.log_dir={tmp_path / 'mr'}"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    logs = sorted((tmp_path / "mr").glob("job_*.log"))
    assert len(logs) == 2 and "JOB 1 a" in logs[0].read_text() and "JOB 2 a" in logs[1].read_text()

    class M:
        logged = None
        def log_dict(self, d): self.logged = d
        @misc.wrap_training_step
        def training_step(self, batch): return {"loss": 1.0, "log": {"lr": 0.1}}
    m = M()
    assert m.training_step(None) == {"loss": 1.0} and m.logged == {"lr": 0.1}
    assert misc.uninject_model_parallel_rank("/a/mp_rank_01/x.ckpt") == "/a/x.ckpt" and misc.uninject_model_parallel_rank("/a/b/x.ckpt") == "/a/b/x.ckpt"
    assert misc.ckpt_to_dir("a/step=10.ckpt") == "a/step=10"
    assert misc.import_class_by_path("collections.OrderedDict").__name__ == "OrderedDict"
    assert misc.parse_dataset_as_name("/data/dev-other_manifest.json") == "dev_other" and misc.parse_dataset_as_name("manifest.json") == "dataset"
    class W:
        def __init__(self, m): self.module = m
    core = object()
    assert misc.unwrap_model(W(W(core))) is core and misc.unwrap_model([W(core)]) == [core]
    from speech_b200.core.modelpt import ModelPT
    from speech_b200 import models  # noqa: F401  (imports the model classes)
    infos = misc.resolve_subclass_pretrained_model_info(ModelPT)
    assert isinstance(infos, list)


def test_run_twice_reports_bitwise_differences_and_guard_bands_catch_overruns():
    from speech_b200.utils.race_check import guarded_empty, run_twice

    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 4)
    x = torch.randn(5, 8)

    def step():
        y = torch.nn.functional.dropout(lin(x), 0.5)          # random, but seeded alike in both runs
        y.sum().backward()
        return {"y": y}

    assert run_twice(step, parameters=list(lin.parameters())).identical
    counter = {"n": 0}

    def racy():
        counter["n"] += 1
        y = lin(x).detach().clone()
        if counter["n"] == 2:
            y[3, 1] += 1e-6                                   # what an unordered accumulation looks like
        return [y]

    rep = run_twice(racy)
    assert not rep.identical and rep.mismatches[0]["name"] == "out[0]" and rep.mismatches[0]["first"] == (3, 1) and rep.mismatches[0]["count"] == 1
    with pytest.raises(AssertionError, match="differ"):
        rep.raise_if_different()

    g = guarded_empty((3, 5), torch.float32, guard_bytes=64, fill=0.0)
    g.tensor.copy_(torch.randn(3, 5))
    g.check()
    flat = g._raw                                             # an out-of-bounds store two floats past the end
    flat[g._guard + 60 + 8] = 0
    assert g.violations() == [("after", 8)]
    with pytest.raises(AssertionError, match="after the payload at byte offset 8"):
        g.check("gemm output")


def test_vad_postprocessing_scoring_and_threshold_tuning(tmp_path):
    import json

    from speech_b200.utils import vad_utils as V

    # window scores -> frame posteriors: a frame covered by three windows gets their mean / median
    w = torch.tensor([0.0, 0.0, 1.0, 1.0, 0.0])
    mean = V.generate_overlap_vad_seq(w, 0.03, 0.01, 0.01, "mean")
    med = V.generate_overlap_vad_seq(w, 0.03, 0.01, 0.01, "median")
    assert mean.shape == (7,) and mean[2] == pytest.approx(1 / 3) and mean[3] == pytest.approx(2 / 3) and float(med[2]) == 0.0 and float(med[3]) == 1.0
    probs = torch.zeros(1000)
    probs[100:300] = 0.9          # 1.0 - 3.0 s
    probs[300:320] = 0.45         # a dip that hysteresis rides through (above offset 0.3)
    probs[320:400] = 0.9          # - 4.0 s
    probs[420:425] = 0.9          # a 50 ms burst
    probs[700:900] = 0.8          # 7.0 - 9.0 s
    seg = V.binarization(probs, {"onset": 0.6, "offset": 0.3, "pad_onset": 0.1, "pad_offset": 0.05})
    assert seg.shape == (3, 2) and seg[0].tolist() == pytest.approx([0.9, 4.05]) and seg[1].tolist() == pytest.approx([4.1, 4.3])
    clean = V.filtering(seg, {"min_duration_on": 0.3, "min_duration_off": 0.2, "filter_speech_first": 1.0})
    assert clean.shape == (2, 2) and clean[1].tolist() == pytest.approx([6.9, 9.05])
    merged = V.filtering(seg, {"min_duration_on": 0.3, "min_duration_off": 0.2, "filter_speech_first": 0.0})
    assert merged[0].tolist() == pytest.approx([0.9, 4.3])                  # gaps filled first: the burst is absorbed
    ref = torch.tensor([[1.0, 4.0], [7.0, 9.0]])
    sc = V.detection_error_rate(ref, torch.tensor([[1.0, 3.0], [7.0, 9.5]]))
    assert sc["miss"] == pytest.approx(20.0) and sc["FA"] == pytest.approx(10.0) and sc["DetER"] == pytest.approx(30.0)
    best, score, trials = V.vad_tune_threshold_on_dev({"onset": [0.3, 0.6, 0.95], "pad_onset": [0.0, 0.5], "min_duration_on": [0.0, 0.2]},
                                                      {"rec": probs}, {"rec": ref})
    assert len(trials) == 12 and best["onset"] in (0.3, 0.6) and best["pad_onset"] == 0.0 and best["min_duration_on"] == 0.2 and score["DetER"] < 1.0
    with pytest.raises(ValueError):
        V.vad_tune_threshold_on_dev({"bogus": [1]}, {"rec": probs}, {"rec": ref})
    labels = torch.zeros(1000)
    labels[100:400] = 1
    labels[700:900] = 1
    assert V.frame_auroc(probs, labels) > 0.98 and V.frame_auroc(torch.rand(1000), labels) == pytest.approx(0.5, abs=0.08)
    rttm = tmp_path / "a.rttm"
    V.write_rttm(str(rttm), ref, "a")
    assert torch.allclose(V.read_rttm_as_segments(str(rttm)), ref)
    assert V.extract_labels(str(rttm), [0.5, 1.5, 5.0, 8.0]) == [0, 1, 0, 1] and V.extract_labels("0 1 1", []) == [0, 1, 1]
    assert V.align_labels_to_frames([0.0] * 6, [0, 1, 1]) == [0, 0, 1, 1, 1, 1] and V.align_labels_to_frames([0.0] * 3, [0, 0, 1, 1, 1, 1]) == [0, 1, 1]
    assert V.convert_labels_to_speech_segments([0, 1, 1, 0, 1], 0.5) == [(0.5, 1.5), (2.0, 2.5)]
    man, out = tmp_path / "m.json", tmp_path / "o.json"
    man.write_text(json.dumps({"audio_filepath": "x.wav", "duration": 950.0}) + "\n" + json.dumps({"audio_filepath": "y.wav", "duration": 30.0}))
    assert V.write_long_audio_manifest(str(man), str(out), split_duration=400.0, window_length_in_sec=0.6) == 4
    rows = [json.loads(l) for l in open(out)]
    assert [r.get("stream_status") for r in rows] == ["start", "next", "end", None] and rows[1]["offset"] == 400.0 and rows[0]["duration"] == 400.6

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.p = torch.nn.Parameter(torch.zeros(1))

        def forward(self, input_signal, input_signal_length):
            e = input_signal.pow(2).mean(dim=1)
            return torch.stack([-(e * 400), e * 400], dim=1) + self.p

    audio = torch.zeros(16000)
    audio[4000:12000] = 0.3 * torch.randn(8000)
    fp = V.generate_vad_frame_pred(Toy(), audio, window_length_in_sec=0.1, shift_length_in_sec=0.02)
    seg = V.generate_vad_segment_table(fp, {"onset": 0.7, "offset": 0.7})
    assert seg.shape == (1, 2) and abs(float(seg[0, 0]) - 0.25) < 0.08 and abs(float(seg[0, 1]) - 0.75) < 0.12


def test_dcp_checkpoint_io_single_process_and_conversion(tmp_path):
    from speech_b200.utils.dcp_io import DCPCheckpointIO, dcp_to_single_file, is_dcp_checkpoint, load_dcp_into_model, single_file_to_dcp

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.Linear(4, 2))
    io = DCPCheckpointIO(async_save=True)
    d = str(tmp_path / "ckpt")
    io.save_checkpoint(dict(model.state_dict(), step=torch.tensor(7)), d, extra={"epoch": 3})
    io.finalize()
    assert is_dcp_checkpoint(d)
    state, extra = io.load_checkpoint(d)
    assert extra == {"epoch": 3} and int(state["step"]) == 7 and torch.equal(state["0.weight"], model[0].weight)
    other = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.Linear(4, 2))
    with pytest.raises(RuntimeError):
        load_dcp_into_model(other, d, strict=True)                              # "step" is not a parameter
    missing, unexpected = load_dcp_into_model(other, d, strict=False)
    assert missing == [] and unexpected == ["step"] and torch.equal(other[1].bias, model[1].bias)
    dcp_to_single_file(d, str(tmp_path / "one.pt"))
    single_file_to_dcp(str(tmp_path / "one.pt"), str(tmp_path / "back"))
    again, extra2 = io.load_checkpoint(str(tmp_path / "back"))
    assert extra2 == {"epoch": 3} and torch.equal(again["1.weight"], model[1].weight)
    tmpl = {k: torch.zeros_like(v) for k, v in model.state_dict().items()}
    io.load_checkpoint(d, template=tmpl)
    assert torch.equal(tmpl["0.bias"], model[0].bias)
    with pytest.raises(ValueError):
        io.load_checkpoint(d, template={"0.weight": torch.zeros(3, 3)})


def test_diarization_and_multispeaker_metrics():
    from speech_b200.models.diarizers import nme_spectral_clustering
    from speech_b200.utils.diar_metrics import (MultiBinaryAccuracy, cp_wer, diarization_error_rate, long_form_clustering, score_labels,
                                                sot_speaker_alignment)

    ref = [(0.0, 10.0, "A"), (10.0, 20.0, "B")]
    # same segmentation with swapped names: the mapping absorbs the swap
    r = diarization_error_rate(ref, [(0.0, 10.0, "x"), (10.0, 20.0, "y")], collar=0.0)
    assert r["DER"] == 0.0 and r["mapping"] == {"x": "A", "y": "B"}
    # boundary placed 2 s late: 2 s of confusion over 20 s; with a 0.25 s collar 0.25 s of it (and 1 s of reference) is not scored
    r = diarization_error_rate(ref, [(0.0, 12.0, "x"), (12.0, 20.0, "y")], collar=0.0)
    assert r["confusion"] == pytest.approx(0.1) and r["miss"] == 0.0 and r["false_alarm"] == 0.0
    r = diarization_error_rate(ref, [(0.0, 12.0, "x"), (12.0, 20.0, "y")], collar=0.25)
    assert r["total"] == pytest.approx(19.0) and r["confusion_time"] == pytest.approx(1.75)
    # a missed stretch, a false alarm, and overlapped speech of which the hypothesis finds one speaker
    ref2 = [(0.0, 10.0, "A"), (8.0, 12.0, "B")]
    hyp2 = [(0.0, 9.0, "x"), (13.0, 14.0, "x")]
    r = diarization_error_rate(ref2, hyp2, collar=0.0)
    assert r["total"] == pytest.approx(14.0) and r["miss_time"] == pytest.approx(1.0 + 4.0) and r["false_alarm_time"] == pytest.approx(1.0)
    r = diarization_error_rate(ref2, hyp2, collar=0.0, ignore_overlap=True)
    assert r["total"] == pytest.approx(10.0) and r["miss_time"] == pytest.approx(2.0)                 # 10-12 s of B alone
    pooled = score_labels({"a": ref, "b": ref2}, {"a": [(0.0, 10.0, "x"), (10.0, 20.0, "y")], "b": hyp2}, collar=0.0, ignore_overlap=False)
    assert pooled["DER"] == pytest.approx(6.0 / 34.0) and pooled["items"]["a"] == 0.0
    score, hyp_order, _ = cp_wer(["good morning all", "hello there my friend"], ["hello there friend", "good morning"])
    assert score == pytest.approx(2 / 5) and hyp_order == ["hello there my friend", "good morning all"]
    assert cp_wer(["a b", "c d", "e"], ["a b", "c d"])[0] == pytest.approx(1 / 4)                      # an extra speaker counts in full
    acc = MultiBinaryAccuracy()
    preds = torch.tensor([[[0.9, 0.1], [0.8, 0.7], [0.2, 0.9], [0.9, 0.9]]])
    tgts = torch.tensor([[[1, 0], [1, 0], [0, 1], [0, 0]]]).float()
    acc.update(preds, tgts, torch.tensor([3]))                                                          # the 4th frame is padding
    f1, prec, rec = acc.compute()
    assert prec == pytest.approx(3 / 4) and rec == 1.0 and acc.accuracy() == pytest.approx(5 / 6)
    import numpy as np

    rng = np.random.default_rng(0)
    cents = rng.standard_normal((3, 16)) * 3
    lab_true = rng.integers(0, 3, 600)
    emb = cents[lab_true] + 0.3 * rng.standard_normal((600, 16))
    cl = lambda aff, mx, oracle: nme_spectral_clustering(aff, mx, oracle)  # noqa: E731
    lab = long_form_clustering(emb, cl, window=200, keep_per_cluster=20, max_num_speakers=4, oracle_num_speakers=3)
    # same partition up to naming
    pairs = {(int(a), int(b)) for a, b in zip(lab_true, lab)}
    assert len(pairs) == 3 and len(set(lab.tolist())) == 3
    score, by = sot_speaker_alignment("hello how are you <sc> fine thanks <sc> good to hear", ["hello how are you good to hear", "fine thanks"])
    assert score == 0.0 and by == ["hello how are you good to hear", "fine thanks"]


def test_asr_evaluation_helpers(tmp_path):
    import json

    from speech_b200.decoding.rnnt_decoding import Hypothesis
    from speech_b200.utils import asr_eval_utils as E

    assert E.clean_label("Hello, [noise] World! It's 42.") == "hello world it's forty two" and E.convert_num_to_words("1205 7") == "one thousand two hundred five seven"
    assert E.strip_spaces_before_punctuations("hi , there !") == "hi, there!" and E.remove_punctuations("a, b. c?") == "a b c"
    man = tmp_path / "p.json"
    man.write_text("\n".join(json.dumps(r) for r in [{"text": "the cat sat", "pred_text": "the cat sat down"}, {"text": "Good Day.", "pred_text": "good day"}]))
    out, wer, ntok, n, rates = E.cal_write_wer(str(man), ignore_capitalization=True, ignore_punctuation=True)
    assert wer == pytest.approx(1 / 5) and (ntok, n) == (5, 2) and rates["ins"] == pytest.approx(1 / 5) and json.loads(open(out).readline())["wer"] == pytest.approx(1 / 3)
    assert E.cal_write_wer(str(man))[1] == pytest.approx(3 / 5)                                       # case and the full stop count
    per = E.PunctuationErrorRate([".", ",", "?"])
    per.update(["Hello, world. how are you", "yes."], ["Hello world. How are you?", "Yes, sure."])
    r = per.compute()
    assert r["."]["correct_rate"] == pytest.approx(0.5) and r[","]["sub_rate"] == pytest.approx(0.5) and r[","]["ins_rate"] == pytest.approx(0.5) and r["?"]["del_rate"] == 1.0
    assert 0 < r["punct_er"] < 1
    # latency: an oracle that emits token i right when 1/gamma more source arrived lags by its constant offset
    assert E.compute_laal([2.0, 3.0, 4.0, 5.0], source_length=4.0, target_length=4) == pytest.approx(2.0)
    assert E.compute_laal([10.0, 10.0], source_length=4.0, target_length=2) == 10.0
    h1 = Hypothesis(score=-1.0, y_sequence=torch.tensor([1, 2]), text="a b", timestamp=[0, 3], token_confidence=[0.9, 0.8])
    h2 = Hypothesis(score=-2.0, y_sequence=torch.tensor([3]), text="c", timestamp=[1], token_confidence=[0.7])
    m = E.merge_parallel_chunks([h1, h2], [10, 8])
    assert m.y_sequence.tolist() == [1, 2, 3] and m.timestamp == [0, 3, 11] and m.text == "a b c" and m.score == -3.0 and m.token_confidence == [0.9, 0.8, 0.7] and m.length == 18
    g = E.merge_hypotheses_of_same_audio([("rec1-1", h2, 8), ("rec1-0", h1, 10), ("rec2_cut0", h2, 8)], decode_tokens_to_str=lambda ids: "".join(map(str, ids)))
    assert g["rec1"].text == "123" and g["rec2"].y_sequence.tolist() == [3]
    h = Hypothesis(score=0.0, y_sequence=[1], timestamp={"word": [{"word": "hi", "start_offset": 5, "end_offset": 9}]})
    E.process_timestamp_outputs([h], subsampling_factor=8, window_stride=0.01)
    assert h.timestamp["word"][0]["start"] == 0.4 and h.timestamp["word"][0]["end"] == 0.72
    assert E.get_ctm_line("utt", 1, 0.5, 0.25, "hello", conf=0.9, speaker="spk1") == "utt 1 0.500 0.250 hello 0.900 lex spk1\n"
    assert E.get_ctm_line("utt", 1, 0.5, 0.25, "hello").endswith("hello NA lex NA\n")
    with pytest.raises(ValueError):
        E.get_ctm_line("u", 1, -1.0, 0.1, "x")
    assert E.get_subsegments(1.0, 2.0, 1.5, 0.75) == [(1.0, 1.5), (1.75, 1.25)]
    rttm = tmp_path / "r.rttm"
    rttm.write_text("SPEAKER r 1 0.0 2.0 <NA> <NA> A <NA> <NA>\nSPEAKER r 1 3.0 1.0 <NA> <NA> B <NA> <NA>\n")
    (tmp_path / "in.json").write_text(json.dumps({"audio_filepath": "/x/r.wav", "rttm_filepath": str(rttm)}))
    assert E.create_segment_manifest(str(tmp_path / "in.json"), str(tmp_path / "seg.json"), window=1.5, shift=0.75) == 3
    d = E.get_subsegment_dict(str(tmp_path / "seg.json"), 1.5, 0.75)
    assert d["r"]["ts"] == [[0.0, 1.5], [0.75, 2.0], [3.0, 4.0]] and d["r"]["json_dic"][2]["label"] == "B"


def test_misc_extra_packing_datastore_dtypes_configs(tmp_path, monkeypatch):
    import dataclasses
    from argparse import ArgumentParser

    from speech_b200.utils import misc_extra as X

    assert X.first_fit([4, 3, 3, 2, 2], 6) == [[4, 2], [3, 3], [2]] and X.first_fit_decreasing([2, 5, 4, 1], 6) == [[5, 1], [4, 2]]
    data = [{"input_ids": list(range(n + 1)), "loss_mask": [0] + [1] * n} for n in (3, 3, 2, 5, 1, 9)]
    by_len, hist = X.create_hist(data, truncate_seq_len=6)
    assert hist == [0, 1, 1, 2, 0, 1, 1] and len(by_len[6]) == 1                                     # the 9-token example was cut to 6
    packs, meta = X.create_packing_strategy(hist, 6, "first_fit_decreasing")
    assert sorted(map(sorted, packs)) == [[1, 5], [2], [3, 3], [6]] and meta["num_packs"] == 4 and meta["packing_factor"] == 1.5
    filled = X.fill_packing_strategy(packs, by_len, 6)
    assert sum(len(f["seq_start_id"]) for f in filled) == 6 and all(len(f["input_ids"]) == len(f["loss_mask"]) for f in filled)
    two = next(f for f in filled if len(f["seq_start_id"]) == 2 and len(f["input_ids"]) == 8)       # lengths 5 and 1 -> 6 + 2 tokens
    assert two["seq_start_id"] == [0, 6]
    monkeypatch.setenv("NEMO_CACHE_DIR", str(tmp_path / "cache"))
    assert X.is_datastore_path("s3://b/k/x.tar") and not X.is_datastore_path("/data/x.tar") and X.is_tarred_path("a/b.tar.gz")
    assert X.bucket_and_object_from_uri("ais://bucket/dir/obj.wav") == ("bucket", "dir/obj.wav")
    calls = []

    def fetch(url, dest):
        calls.append(url)
        open(dest, "w").write("payload")

    obj = X.DataStoreObject("s3://b/k/x.txt", fetch=fetch)
    assert obj.local_path == str(tmp_path / "cache" / "datastore" / "s3" / "b" / "k" / "x.txt") and obj.local_path and len(calls) == 1
    assert X.open_best("s3://b/k/x.txt", "r", fetch=fetch).read() == "payload" and len(calls) == 1    # cached
    with pytest.raises(RuntimeError):
        X.DataStoreObject("gs://nobody/registered").get()
    assert X.str_to_dtype("bf16-mixed") is torch.bfloat16 and X.str_to_dtype(16) is torch.float16 and X.str_to_dtype(torch.float64) is torch.float64
    with pytest.raises(ValueError):
        X.str_to_dtype("int3")
    m = X.CastToFloat(torch.nn.Softmax(dim=-1))
    y = m(torch.randn(2, 5, dtype=torch.bfloat16))
    assert y.dtype == torch.bfloat16
    out = X.CastToFloatAll(torch.nn.Bilinear(3, 3, 2))(torch.randn(4, 3, dtype=torch.float16), torch.randn(4, 3, dtype=torch.float16))
    assert out.dtype == torch.float16
    with X.monkeypatched(torch, "is_tensor", lambda x: "patched"):
        assert torch.is_tensor(1) == "patched"
    assert torch.is_tensor(torch.zeros(1)) is True and X.maybe_cast_to_type("3", int) == 3 and X.maybe_cast_to_type(None, int) is None

    @dataclasses.dataclass
    class Schema:
        sample_rate: int = 16000
        train_ds: dict = dataclasses.field(default_factory=lambda: {"batch_size": 8, "shuffle": True})
        validation_ds: dict = dataclasses.field(default_factory=lambda: {"batch_size": 8})

    cfg = X.update_model_config(Schema(), {"sample_rate": 8000, "train_ds": {"batch_size": 4, "extra": 1}})
    assert cfg.sample_rate == 8000 and cfg.train_ds.batch_size == 4 and cfg.train_ds.shuffle and cfg.train_ds.extra == 1 and "validation_ds" not in cfg

    class Mod:
        def __init__(self, sample_rate, hidden, legacy=None):
            pass

    @dataclasses.dataclass
    class ModCfg:
        sample_rate: int = 1
        width: int = 2

    assert X.assert_dataclass_signature_match(Mod, ModCfg, ignore_args=["legacy"], remap_args={"hidden": "width"}) == (True, None, None)
    assert X.assert_dataclass_signature_match(Mod, ModCfg)[1] == {"hidden", "legacy"}
    src = tmp_path / "a.txt"
    src.write_text("x")
    fails = {"n": 0}

    def flaky(s, d):
        fails["n"] += 1
        if fails["n"] < 3:
            raise OSError("stale handle")
        import shutil

        shutil.copy2(s, d)

    assert X.robust_copy(src, tmp_path / "b.txt", retries=3, backoff=0.0, copy_fn=flaky).endswith("b.txt") and fails["n"] == 3
    p = X.add_asr_args(X.add_scheduler_args(X.add_optimizer_args(ArgumentParser(), default_lr=1e-3)))
    a = p.parse_args(["--asr_model", "m", "--train_dataset", "t", "--eval_dataset", "e", "--opt_args", "betas=0.9,0.98"])
    assert a.lr == 1e-3 and a.opt_args == ["betas=0.9,0.98"] and a.min_lr == 0.0
