"""The example scripts run end to end: train a tiny CTC model from the shipped YAML, then transcribe with the saved .nemo,
then stream the same files through the buffered pipeline script."""
import glob
import json
import os
import subprocess
import sys

import numpy as np

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, args, cwd):
    env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, os.path.join(REPO, script)] + args, cwd=cwd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]
    return out.stdout + out.stderr


def test_train_transcribe_and_stream_examples(tmp_path):
    from speech_b200.data.audio_to_text import save_wav

    g = np.random.default_rng(0)
    man = tmp_path / "test.json"
    with open(man, "w") as f:
        for i in range(3):
            p = str(tmp_path / f"a{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(16000 + 3000 * i)).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 1.0 + 0.1875 * i, "text": "w1 w2"}) + "\n")
    exp = tmp_path / "exp"
    _run("examples/asr/asr_ctc/speech_to_text_ctc_bpe.py", [
        "model.tokenizer.type=synthetic", "+model.tokenizer.vocab_size=32", "model.tokenizer.dir=null",
        "+model.train_ds.synthetic={num_samples: 8, vocab_size: 32, min_duration: 1.0, max_duration: 1.5}",
        "model.train_ds.manifest_filepath=null", "model.validation_ds.manifest_filepath=null", "model.train_ds.batch_size=4",
        "model.train_ds.num_workers=0", "model.encoder.n_layers=1", "model.encoder.d_model=64", "model.encoder.n_heads=4",
        "trainer.max_steps=2", "trainer.max_epochs=null", "trainer.accelerator=cpu", "trainer.devices=1", "trainer.precision=32",
        "trainer.strategy=auto", f"exp_manager.exp_dir={exp}", "exp_manager.create_tensorboard_logger=false"], str(tmp_path))
    nemo = glob.glob(str(exp / "**" / "*.nemo"), recursive=True)
    assert nemo
    out_json = tmp_path / "out.json"
    log = _run("examples/asr/transcribe_speech.py", [f"model_path={nemo[0]}", f"dataset_manifest={man}", f"output_filename={out_json}",
                                                     "batch_size=2", "cuda=-1", "calculate_rtfx=true"], str(tmp_path))
    recs = [json.loads(l) for l in open(out_json)]
    assert len(recs) == 3 and all("pred_text" in r for r in recs) and "RTFx" in log
    log = _run("examples/asr/asr_streaming_inference/asr_streaming_infer.py", [
        "--config-name", "buffered_ctc", f"asr.model_name={nemo[0]}", "asr.device=cpu", "asr.compute_dtype=float32", f"audio_file={man}",
        f"output_filename={tmp_path / 'stream.json'}", "streaming.batch_size=2", "streaming.chunk_size=0.4",
        "streaming.left_padding_size=0.4", "streaming.right_padding_size=0.2"], str(tmp_path))
    assert "RTFx" in log and len(open(tmp_path / "stream.json").read().splitlines()) == 3


def test_adapter_training_and_evaluation_examples(tmp_path):
    """Base model from the CTC example, then the adapter recipe: only the adapter trains, it is saved alone and with the model, and
    the evaluation script reports WER with and without it."""
    import torch
    from speech_b200.data.audio_to_text import save_wav

    g = np.random.default_rng(0)
    man = tmp_path / "train.json"
    with open(man, "w") as f:
        for i in range(4):
            p = str(tmp_path / f"a{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(16000)).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 1.0, "text": "w1 w2 w3"}) + "\n")
    exp = tmp_path / "exp"
    _run("examples/asr/asr_ctc/speech_to_text_ctc_bpe.py", [
        "model.tokenizer.type=synthetic", "+model.tokenizer.vocab_size=32", "model.tokenizer.dir=null",
        "+model.train_ds.synthetic={num_samples: 4, vocab_size: 32, min_duration: 1.0, max_duration: 1.2}",
        "model.train_ds.manifest_filepath=null", "model.validation_ds.manifest_filepath=null", "model.train_ds.batch_size=4",
        "model.train_ds.num_workers=0", "model.encoder.n_layers=1", "model.encoder.d_model=64", "model.encoder.n_heads=4",
        "trainer.max_steps=1", "trainer.max_epochs=null", "trainer.accelerator=cpu", "trainer.devices=1", "trainer.precision=32",
        "trainer.strategy=auto", f"exp_manager.exp_dir={exp}", "exp_manager.create_tensorboard_logger=false"], str(tmp_path))
    base = glob.glob(str(exp / "**" / "*.nemo"), recursive=True)[0]
    out = tmp_path / "adapt"
    _run("examples/asr/asr_adapters/train_asr_adapter.py", [
        f"model.nemo_model={base}", f"model.train_ds.manifest_filepath={man}", "model.train_ds.batch_size=2", "model.train_ds.max_duration=5.0",
        "model.adapter.adapter_name=encoder:domain", "model.adapter.d_model=64", "model.adapter.linear.dim=4", "model.optim.sched=null",
        "trainer.max_steps=2", "trainer.accelerator=cpu", "trainer.precision=32", f"exp_manager.exp_dir={out}",
        "+exp_manager.create_tensorboard_logger=false"], str(tmp_path))
    ad = glob.glob(str(out / "**" / "adapters.pt"), recursive=True)
    adapted = glob.glob(str(out / "**" / "ASR-Adapter.nemo"), recursive=True)
    assert ad and adapted
    blob = torch.load(ad[0], weights_only=False)
    assert list(blob["__cfg__"]) == ["encoder:domain"] and all("adapter_layer.domain" in k for k in blob["state_dict"])
    log = _run("examples/asr/asr_adapters/eval_asr_adapter.py", [f"model_path={adapted[0]}", f"manifest={man}", "adapter_name=encoder:domain", "batch_size=2"],
               str(tmp_path))
    res = json.loads([l for l in log.splitlines() if l.startswith("{")][-1])
    assert res["enabled_adapters"] == ["encoder:domain"] and "wer_with_adapter" in res and "wer_without_adapters" in res


def test_aed_trains_from_a_manifest_with_prompts_and_the_chunked_and_streaming_scripts_run(tmp_path):
    import torch
    from speech_b200.core.trainer import Trainer
    from speech_b200.data.audio_to_text import save_wav
    from speech_b200.models import EncDecMultiTaskModel
    from speech_b200.models.configs import canary_aed_config

    g = np.random.default_rng(0)
    man = tmp_path / "train.json"
    with open(man, "w") as f:
        for i in range(4):
            p = str(tmp_path / f"a{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(16000 + 4000 * i)).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 1.0 + 0.25 * i, "text": "ab cd", "lang": "en", "source_lang": "en",
                                "target_lang": "de" if i % 2 else "en", "pnc": "no"}) + "\n")
    specials = ["<|nospeech|>", "<pad>", "<|endoftext|>", "<|startoftranscript|>", "<|pnc|>", "<|nopnc|>", "<|transcribe|>", "<|translate|>",
                "<|en|>", "<|de|>"]
    letters = list("abcdefghijklmnopqrstuvwxyz ")
    tok = {"type": "agg", "langs": {"spl_tokens": {"type": "char", "vocab": specials}, "en": {"type": "char", "vocab": letters},
                                    "de": {"type": "char", "vocab": letters}}}
    cfg = canary_aed_config("small", enc_layers=1, dec_layers=1, dec_hidden=64, dec_heads=4, dec_inner=128, vocab_size=64, features=32,
                            dropout=0.0, max_sequence_length=128, tokenizer=tok)
    from speech_b200.core.config import open_dict
    with open_dict(cfg):
        cfg.prompt_format = "canary"
        cfg.train_ds = {"manifest_filepath": str(man), "batch_size": 2, "shuffle": False, "sample_rate": 16000}
    m = EncDecMultiTaskModel(cfg)
    batch = next(iter(m._train_dl))
    assert len(batch) == 6 and batch[2].shape[0] == 2 and batch[5].tolist() == [5, 5]           # five prompt tokens per utterance
    sid = m.tokenizer.spl_token_to_id
    assert batch[4][1].tolist() == [sid("startoftranscript"), sid("en"), sid("translate"), sid("de"), sid("nopnc")]
    tr = Trainer(max_steps=2, accelerator="cpu", enable_checkpointing=False, logger=False, log_every_n_steps=1)
    tr.fit(m)
    assert np.isfinite(float(tr.callback_metrics["train_loss"]))
    nemo = str(tmp_path / "aed.nemo")
    m.save_to(nemo)
    out = tmp_path / "chunked.json"
    _run("examples/asr/asr_chunked_inference/aed/speech_to_text_aed_chunked_infer.py",
         [f"model_path={nemo}", f"dataset_manifest={man}", f"output_filename={out}", "chunk_len_in_secs=0.6", "batch_size=2"], str(tmp_path))
    recs = [json.loads(l) for l in open(out)]
    assert len(recs) == 4 and all("pred_text" in r for r in recs)
    out2 = tmp_path / "stream.json"
    _run("examples/asr/asr_chunked_inference/aed/speech_to_text_aed_streaming_infer.py",
         [f"model_path={nemo}", f"dataset_manifest={man}", f"output_filename={out2}", "chunk_secs=0.4", "decoding.streaming_policy=alignatt",
          "decoding.alignatt_thr=2"], str(tmp_path))
    recs = [json.loads(l) for l in open(out2)]
    assert len(recs) == 4 and all("average_lagging_s" in r for r in recs)


def test_duplex_infer_example_and_mesh_strategy_from_yaml(tmp_path):
    import torch
    from speech_b200.core.config import OmegaConf
    from speech_b200.data.audio_to_text import save_wav
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.parallel.strategy import ParallelStrategy
    from speech_b200.speechlm.duplex import DuplexSTTModel
    from speech_b200.utils.launch import build_trainer

    tr = build_trainer(OmegaConf.create({"trainer": {"accelerator": "cpu", "max_steps": 1, "strategy": {"dp_shard_size": -1, "tp_size": 1,
                                                                                                    "sequence_parallel": False}}}))
    assert isinstance(tr.strategy_spec, ParallelStrategy) and tr.strategy_spec.dp_shard_size == -1
    for name in ("salm_automodel", "duplex_stt", "salm"):
        assert OmegaConf.load(os.path.join(REPO, "examples", "speechlm2", "conf", name + ".yaml")).model is not None
    torch.manual_seed(0)
    tiny = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                head_dim=8, tie_word_embeddings=True, qk_norm=True, model_type="qwen3")
    pc = {"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}
    m = DuplexSTTModel(OmegaConf.create({"llm": tiny, "perception": pc, "predict_user_text": True, "optim": {"name": "adamw", "lr": 1e-3}}))
    nemo = str(tmp_path / "duplex.nemo")
    m.save_to(nemo)
    g = np.random.default_rng(0)
    man = tmp_path / "in.json"
    with open(man, "w") as f:
        for i in range(2):
            p = str(tmp_path / f"d{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(16000)).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 1.0, "user_end_time": 0.8}) + "\n")
    out = tmp_path / "gen.jsonl"
    log = _run("examples/speechlm2/stt_duplex_infer.py", [f"pretrained_name={nemo}", f"inputs={man}", f"output_manifest={out}", "pad_seconds=0.5",
                                                          "device=cpu", "batch_size=2"], str(tmp_path))
    recs = [json.loads(l) for l in open(out)]
    assert len(recs) == 2 and all("pred_text" in r and "pred_user_text" in r for r in recs) and "turn taking" in log


def test_tts_training_examples_run_through_the_trainer(tmp_path):
    """FastPitch, the aligner, HiFi-GAN and the codec train from their shipped YAML on synthetic tone data; the adversarial
    models go through the trainer's manual optimisation (generator and discriminator updated in turn)."""
    common = ["trainer.max_steps=2", "trainer.max_epochs=null", "trainer.accelerator=cpu", "trainer.devices=1", "trainer.strategy=auto",
              "exp_manager.create_tensorboard_logger=false", "exp_manager.create_checkpoint_callback=false", "model.train_ds.manifest_filepath=null",
              "model.sample_rate=8000"]
    syn = "+model.train_ds.synthetic={num_samples: 4, min_chars: 3, max_chars: 5}"
    small_tf = ["model.symbols_embedding_dim=32", "model.d_inner=64", "model.encoder_layers=1", "model.decoder_layers=1", "model.n_mel_channels=20",
                "model.n_fft=256", "model.hop_length=64", "model.win_length=256", "model.train_ds.batch_size=2", "model.train_ds.num_workers=0"]
    _run("examples/tts/fastpitch.py", common + small_tf + [syn, f"exp_manager.exp_dir={tmp_path / 'fp'}", "model.optim.sched.warmup_steps=1"], str(tmp_path))
    assert os.path.isdir(tmp_path / "fp" / "FastPitch")
    _run("examples/tts/aligner.py", common + [syn, "model.symbols_embedding_dim=16", "model.n_mel_channels=20", "model.mel={n_fft: 256, hop: 64, win: 256}",
                                              "model.train_ds.batch_size=2", "model.train_ds.num_workers=0", f"exp_manager.exp_dir={tmp_path / 'al'}"], str(tmp_path))
    _run("examples/tts/hifigan.py", common + [syn, "model.generator={input_dim: 20, up_sample_rates: [4, 4, 4], base_channels: 16, resblock_kernel_sizes: [3]}",
                                              "model.discriminator={periods: [2], stft_resolutions: [[256, 64, 256]]}", "model.mel={n_fft: 256, hop: 64, win: 256}",
                                              "model.train_ds.batch_size=2", "model.train_ds.num_workers=0", f"exp_manager.exp_dir={tmp_path / 'hg'}"], str(tmp_path))


def test_hybrid_conversion_evaluation_finetune_and_speaker_examples(tmp_path):
    from speech_b200.data.audio_to_text import save_wav

    g = np.random.default_rng(0)
    man = tmp_path / "test.json"
    with open(man, "w") as f:
        for i in range(3):
            p = str(tmp_path / f"a{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(16000 + 3000 * i)).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 1.0 + 0.1875 * i, "text": "w1 w2"}) + "\n")
    small = ["model.tokenizer.type=synthetic", "+model.tokenizer.vocab_size=32", "model.tokenizer.dir=null",
             "+model.train_ds.synthetic={num_samples: 4, vocab_size: 32, min_duration: 1.0, max_duration: 1.2}", "model.train_ds.manifest_filepath=null",
             "model.validation_ds.manifest_filepath=null", "model.train_ds.batch_size=4", "model.train_ds.num_workers=0", "model.encoder.n_layers=1",
             "model.encoder.d_model=64", "model.encoder.n_heads=4", "model.model_defaults.enc_hidden=64", "trainer.max_steps=1", "trainer.max_epochs=null",
             "trainer.accelerator=cpu", "trainer.devices=1", "trainer.precision=32", "trainer.strategy=auto", "exp_manager.create_tensorboard_logger=false"]
    _run("examples/asr/asr_hybrid_transducer_ctc/speech_to_text_hybrid_rnnt_ctc_bpe.py", small + [f"exp_manager.exp_dir={tmp_path / 'exp'}"], str(tmp_path))
    hybrid = glob.glob(str(tmp_path / "exp" / "**" / "*.nemo"), recursive=True)[0]
    ctc = str(tmp_path / "ctc.nemo")
    _run("examples/asr/asr_hybrid_transducer_ctc/helpers/convert_nemo_asr_hybrid_to_ctc.py", ["-i", hybrid, "-o", ctc, "-t", "ctc"], str(tmp_path))
    assert os.path.getsize(ctc) < os.path.getsize(hybrid)                      # the prediction and joint networks are gone
    log = _run("examples/asr/speech_to_text_eval.py", [f"model_path={ctc}", f"dataset_manifest={man}", f"output_filename={tmp_path / 'eval.json'}", "cuda=-1",
                                                       "scores_per_sample=true", "text_processing.do_lowercase=true"], str(tmp_path))
    rows = [json.loads(l) for l in open(tmp_path / "eval.json")]
    assert "WER:" in log and len(rows) == 3 and all("pred_text" in r and "wer" in r for r in rows)
    log = _run("examples/asr/speech_to_text_eval.py", [f"dataset_manifest={tmp_path / 'eval.json'}", "only_score_manifest=true", "tolerance=1000",
                                                       f"output_filename={tmp_path / 'eval2.json'}"], str(tmp_path))
    assert "WER:" in log
    _run("examples/asr/speech_to_text_finetune.py", [f"init_from_nemo_model={ctc}", "model.train_ds={manifest_filepath: " + str(man) + ", batch_size: 2, shuffle: true, "
                                                     "num_workers: 0, max_duration: 5.0}", "trainer.max_steps=2", "trainer.accelerator=cpu",
                                                     f"exp_manager.exp_dir={tmp_path / 'ft'}"], str(tmp_path))
    _run("examples/asr/asr_vad/speech_to_text_with_vad.py", [f"asr_model={ctc}", "use_energy_vad=true", f"manifest_filepath={man}",
                                                             f"output_filename={tmp_path / 'vadasr.json'}", "cuda=-1"], str(tmp_path))
    assert len(open(tmp_path / "vadasr.json").read().splitlines()) == 3

    # speaker pipeline: train -> embeddings -> trial scoring -> identification
    t = np.arange(16000) / 16000
    rows = []
    for spk, f0 in (("A", 150), ("B", 300)):
        os.makedirs(tmp_path / "spk" / spk / "s")
        for i in range(3):
            p = str(tmp_path / "spk" / spk / "s" / f"u{i}.wav")
            save_wav(p, (0.3 * np.sin(2 * np.pi * f0 * t) + 0.02 * g.standard_normal(16000)).astype(np.float32))
            rows.append({"audio_filepath": p, "duration": 1.0, "label": spk})
    dump = lambda name, rs: open(tmp_path / name, "w").write("\n".join(json.dumps(r) for r in rs))  # noqa: E731
    dump("spk_train.json", rows)
    dump("enroll.json", [r for r in rows if not r["audio_filepath"].endswith("u2.wav")])
    dump("spk_test.json", [r for r in rows if r["audio_filepath"].endswith("u2.wav")])
    tr = [r["audio_filepath"] for r in rows]
    open(tmp_path / "trials.txt", "w").write(f"1 {tr[0]} {tr[1]}\n0 {tr[0]} {tr[3]}\n1 {tr[3]} {tr[4]}\n0 {tr[2]} {tr[5]}\n")
    _run("examples/speaker_tasks/recognition/speaker_reco.py", [
        f"model.train_ds.manifest_filepath={tmp_path / 'spk_train.json'}", f"model.validation_ds.manifest_filepath={tmp_path / 'spk_train.json'}",
        "model.train_ds.batch_size=6", "model.validation_ds.batch_size=6", "model.train_ds.num_workers=0", "model.validation_ds.num_workers=0",
        "model.decoder.num_classes=2", "trainer.max_steps=10", "trainer.max_epochs=null", "trainer.accelerator=cpu", "trainer.devices=1", "trainer.strategy=auto",
        "trainer.precision=32", f"exp_manager.exp_dir={tmp_path / 'spkexp'}", "exp_manager.create_tensorboard_logger=false"], str(tmp_path))
    spk = glob.glob(str(tmp_path / "spkexp" / "**" / "*.nemo"), recursive=True)[0]
    out = _run("examples/speaker_tasks/recognition/extract_speaker_embeddings.py", [f"--manifest={tmp_path / 'spk_train.json'}", f"--model_path={spk}",
                                                                                      f"--embedding_dir={tmp_path / 'emb'}"], str(tmp_path))
    pkl = str(tmp_path / "emb" / "embeddings" / "spk_train_embeddings.pkl")
    assert pkl in out
    out = _run("examples/speaker_tasks/recognition/voxceleb_eval.py", [f"--trial_file={tmp_path / 'trials.txt'}", f"--emb={pkl}"], str(tmp_path))
    assert "EER:" in out and "minDCF:" in out                # the 10-step model's quality is not the subject here
    import importlib.util

    spec = importlib.util.spec_from_file_location("voxceleb_eval", os.path.join(REPO, "examples/speaker_tasks/recognition/voxceleb_eval.py"))
    sys.path.insert(0, os.path.join(REPO, "examples/speaker_tasks/recognition"))
    try:
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        sys.path.pop(0)
    eer, dcf = mod.eer_and_min_dcf(np.array([0.9, 0.8, 0.7, 0.3, 0.2, 0.1]), np.array([1, 1, 1, 0, 0, 0]))
    assert eer == 0.0 and dcf == 0.0
    eer, _ = mod.eer_and_min_dcf(np.array([0.9, 0.8, 0.3, 0.7, 0.2, 0.1]), np.array([1, 1, 1, 0, 0, 0]))
    assert abs(eer - 1 / 3) < 1e-9
    for backend in ("cosine_similarity", "neural_classifier"):
        out = _run("examples/speaker_tasks/recognition/speaker_identification_infer.py", [
            f"model_path={spk}", f"data.enrollment_manifest={tmp_path / 'enroll.json'}", f"data.test_manifest={tmp_path / 'spk_test.json'}",
            f"data.out_manifest={tmp_path / ('id_' + backend + '.json')}", f"backend.backend_model={backend}", "cuda=-1"], str(tmp_path))
        assert "accuracy:" in out and len(open(tmp_path / ("id_" + backend + ".json")).read().splitlines()) == 2


def test_voice_agent_stream_parsers_and_websocket_url():
    import importlib.util

    def load(rel):
        spec = importlib.util.spec_from_file_location(os.path.basename(rel)[:-3], os.path.join(REPO, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    rp = load("examples/voice_agent/server/parsers/reasoning_parser.py")
    text = "<think>the user greets me</think>Hello! <think>short</think>How are you?"
    for size in (1, 3, 7, len(text)):                      # any chunking, tags cut in the middle included
        p = rp.StreamingReasoningParser()
        r = c = ""
        for i in range(0, len(text), size):
            d = p.feed(text[i:i + size])
            r, c = r + d.reasoning, c + d.content
        d = p.flush()
        assert (r + d.reasoning, c + d.content) == ("the user greets meshort", "Hello! How are you?"), size
    assert rp.split_reasoning("planning...</think>Answer") == ("planning...", "Answer")       # closing tag without an opening one
    assert rp.split_reasoning("a < b and x <thin air") == (None, "a < b and x <thin air")
    tp = load("examples/voice_agent/server/parsers/toolcall_parser_streaming.py")
    text = 'Let me check. <TOOLCALL>[{"name": "weather", "arguments": {"city": "Paris {FR}", "note": "say \\"hi\\""}}, {"name": "time", "arguments": "{\\"tz\\": \\"CET\\"}"}]</TOOLCALL> Done.'
    for size in (1, 5, 11, len(text)):
        p = tp.StreamingToolCallParser()
        content, calls, first_call_at = "", [], None
        for i in range(0, len(text), size):
            d = p.feed(text[i:i + size])
            content += d.content
            if d.tool_calls and first_call_at is None:
                first_call_at = i
            calls += d.tool_calls
        d = p.flush()
        content += d.content
        assert content == "Let me check.  Done." and [c["function"]["name"] for c in calls] == ["weather", "time"], size
        assert calls[0]["function"]["arguments"] == {"city": "Paris {FR}", "note": 'say "hi"'} and calls[1]["function"]["arguments"] == {"tz": "CET"}
        assert [c["id"] for c in calls] == ["call_0", "call_1"]
        if size == 1:
            assert first_call_at < text.index('{"name": "time"')          # the first call is out before the second one is complete
    p = tp.StreamingToolCallParser()
    p.feed('<TOOLCALL>[{"name": "x", "arguments": {"a": 1')
    assert p.flush().errors
    wu = load("examples/voice_agent/server/websocket_url.py")
    assert wu.websocket_url("0.0.0.0", 7860) == "ws://localhost:7860/ws"
    assert wu.websocket_url("0.0.0.0", 7860, headers={"Host": "demo.example.com", "X-Forwarded-Proto": "https", "X-Forwarded-Prefix": "/agent/"}) == "wss://demo.example.com/agent/ws"
    assert wu.websocket_url("::1", 9000, path="/audio") == "ws://[::1]:9000/audio"
    assert wu.websocket_url("0.0.0.0", 1, public_url="https://x.example.org/base") == "wss://x.example.org/base/ws"


def test_g2p_and_ssl_tts_examples(tmp_path):
    lex = [("cat", "k æ t"), ("tack", "t æ k"), ("act", "æ k t"), ("box", "b ɑ k s"), ("tax", "t æ k s"), ("cab", "k æ b")]
    (tmp_path / "train.json").write_text("\n".join(json.dumps({"text_graphemes": g_, "text": p}, ensure_ascii=False) for g_, p in lex), encoding="utf-8")
    (tmp_path / "phones.txt").write_text("\n".join(sorted({x for _, p in lex for x in p.split()})), encoding="utf-8")
    ds = "{manifest_filepath: " + str(tmp_path / "train.json") + ", batch_size: 6}"
    log = _run("examples/tts/g2p/g2p_train_and_evaluate.py", ["model_type=ctc", f"model.phonemes={tmp_path / 'phones.txt'}", f"model.train_ds={ds}", f"model.validation_ds={ds}",
                                                               f"model.test_ds={ds}", "do_testing=true", "model.d_model=32", "model.n_layers=1", "model.n_heads=2",
                                                               "model.optim.lr=0.005", "trainer.max_epochs=150", "trainer.accelerator=cpu", f"exp_manager.exp_dir={tmp_path / 'exp'}"],
               str(tmp_path))
    assert "test PER" in log
    nemo = glob.glob(str(tmp_path / "exp" / "**" / "*.nemo"), recursive=True)[0]
    log = _run("examples/tts/g2p/g2p_inference.py", [f"pretrained_model={nemo}", f"manifest_filepath={tmp_path / 'train.json'}", f"output_file={tmp_path / 'out.json'}"],
               str(tmp_path))
    assert "PER:" in log and float(log.split("PER:")[1].split()[0]) < 0.2
    assert "pred_text" in json.loads(open(tmp_path / "out.json", encoding="utf-8").readline())
    _run("examples/tts/ssl_tts.py", ["+model.train_ds.synthetic={num_samples: 4}", "model.train_ds.manifest_filepath=null", "model.train_ds.batch_size=2",
                                     "model.train_ds.num_workers=0", "model.encoder.n_layers=1", "model.encoder.d_model=32", "model.encoder.n_heads=2", "model.encoder_dim=32",
                                     "model.encoder.subsampling_conv_channels=16", "trainer.max_steps=2", "trainer.max_epochs=null", "trainer.accelerator=cpu", "trainer.devices=1",
                                     "trainer.strategy=auto", f"exp_manager.exp_dir={tmp_path / 'ssl'}", "exp_manager.create_tensorboard_logger=false"], str(tmp_path))


def test_adapter_sweep_scoring_picks_constrained_and_unconstrained_winners(tmp_path):
    import importlib.util
    import itertools
    import json

    import pandas as pd

    spec = importlib.util.spec_from_file_location("scoring_and_analysis", os.path.join(REPO, "examples", "asr", "asr_adapters", "scoring_and_analysis.py"))
    sa = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sa)
    rows = []
    for pos, dim, g in itertools.product(["encoder", "decoder"], [32, 64], ["a", "b"]):
        rows.append({"Adapter Position": pos, "Adapter Dimensions": dim, "Adapter Dropout": 0.1, "Stochastic Depth": 0.0, "Train Steps": 1000, "Dataset": g,
                     "WER: Test": 10 - (2 if dim == 64 else 1) - (1 if pos == "encoder" else 0), "WER: Original Test": 5 + (4 if dim == 64 else 0.5)})
    pd.DataFrame(rows).to_csv(tmp_path / "sweep.csv", index=False)
    (tmp_path / "base.json").write_text(json.dumps({"original": 5.0, "adapted": {"a": 10.0, "b": 10.0}}))
    best = sa.main(["--csv", str(tmp_path / "sweep.csv"), "--dataset_type_column", "Dataset", "--baselines", str(tmp_path / "base.json")])
    assert [b["Adapter Dimensions"] for b in best] == [64, 64, 32, 32]     # lowest WER wins unconstrained; the run that ruins the original domain scores 0
    df = pd.read_csv(tmp_path / "sweep.csv")
    assert abs(df[(df["Adapter Dimensions"] == 32) & (df["Adapter Position"] == "encoder")]["Score"].iloc[0] - (2.5 / 3) * 0.2) < 1e-3
    only = sa.main(["--csv", str(tmp_path / "sweep.csv"), "--dataset_type_column", "Dataset", "--baselines", str(tmp_path / "base.json"), "-uargs", "Adapter Dimensions", "32"])
    assert only[0]["Adapter Dimensions"] == 32
    assert sa.original_scale(9.0, 5.0, 3.0) == 0.0 and sa.adapt_werr(12.0, 10.0) == 0.0
