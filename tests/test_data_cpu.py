"""Cut-based data pipeline on CPU: manifests and tarred shards, input_cfg mux, filters, speed perturbation, bucketing
(1-D, 2-D, token budget), noise / RIR augmentation, multi-config fusion, rank sharding."""
import io
import json
import os
import tarfile

import numpy as np
import pytest
import torch

from speech_b200.data.audio_to_text import save_wav
from speech_b200.data.cuts import (Cut, CutSet, NoiseMixer, RIRConvolver, determine_bucket_duration_bins,
                                   get_dataloader_from_cuts_config, parse_input_cfg, read_nemo_manifest, speed_perturb)
from speech_b200.tokenizers import CharTokenizer

TOK = CharTokenizer(list("abcdefghijklmnopqrstuvwxyz "))


def _corpus(tmp_path, n=12, name="m"):
    g = np.random.default_rng(0)
    items = []
    for i in range(n):
        d = 0.2 + 0.1 * i
        p = str(tmp_path / f"{name}{i}.wav")
        save_wav(p, (0.1 * g.standard_normal(int(16000 * d))).astype(np.float32))
        items.append({"audio_filepath": p, "duration": d, "text": "ab " * (1 + i % 4), "lang": "en"})
    man = str(tmp_path / f"{name}.json")
    with open(man, "w") as f:
        for it in items:
            f.write(json.dumps(it) + "\n")
    return man, items


def test_manifest_filters_buckets_and_rank_sharding(tmp_path):
    man, items = _corpus(tmp_path)
    cfg = {"manifest_filepath": man, "use_lhotse": True, "batch_duration": 2.0, "num_buckets": 2, "min_duration": 0.3,
           "max_duration": 1.2, "shuffle": True, "seed": 1, "perturb_speed": False}
    seen = []
    for rank in range(2):
        dl = get_dataloader_from_cuts_config(cfg, rank, 2, tokenizer=TOK)
        for audio, alen, tok, tlen in dl:
            assert audio.shape[0] == alen.numel() and float(alen.max()) / 16000 * len(alen) <= 2.0 + 1e-6
            seen.append(sorted(alen.tolist()))
    flat = sorted(x for b in seen for x in b)
    kept = [int(16000 * it["duration"]) for it in items if 0.3 <= it["duration"] <= 1.2]
    assert len(flat) <= len(kept) and set(flat) <= set(kept)
    assert len(seen) % 2 == 0                        # both ranks got the same number of batches


def test_input_cfg_mux_weights_tags_and_speed_perturbation(tmp_path):
    m1, _ = _corpus(tmp_path, 6, "a")
    m2, _ = _corpus(tmp_path, 6, "b")
    cuts = parse_input_cfg([{"type": "nemo", "manifest_filepath": m1, "weight": 0.9, "tags": {"src": "a"}},
                            {"type": "group", "weight": 0.1, "input_cfg": [{"type": "nemo", "manifest_filepath": m2, "tags": {"src": "b"}}]}],
                           seed=3)
    srcs = [c.custom["src"] for c in cuts]
    assert sorted(srcs) == ["a"] * 6 + ["b"] * 6 and srcs[:4].count("a") >= 3
    c = next(iter(read_nemo_manifest(m1)))
    fast = c.with_speed(1.1)
    assert abs(fast.duration - c.duration / 1.1) < 1e-9 and abs(len(fast.load_audio()) - len(c.load_audio()) / 1.1) <= 2
    x = np.sin(np.arange(1600) * 0.1).astype(np.float32)
    assert len(speed_perturb(x, 0.9)) == round(1600 / 0.9)
    dl = get_dataloader_from_cuts_config({"input_cfg": [{"type": "nemo", "manifest_filepath": m1}], "batch_size": 4,
                                          "perturb_speed": [0.9, 1.1]}, tokenizer=TOK)
    assert sum(b[0].shape[0] for b in dl) == 18


def test_two_dim_buckets_token_budget_and_duration_bins(tmp_path):
    man, items = _corpus(tmp_path)
    dl = get_dataloader_from_cuts_config({"manifest_filepath": man, "use_lhotse": True,
                                          "bucket_duration_bins": [[0.6, 6], [0.6, 12], [1.4, 6], [1.4, 12]],
                                          "bucket_batch_size": [4, 3, 2, 1]}, tokenizer=TOK)
    for audio, alen, tok, tlen in dl:
        d, t = float(alen.max()) / 16000, int(tlen.max())
        limit = 4 if (d <= 0.6 and t <= 6) else 3 if d <= 0.6 else 2 if t <= 6 else 1
        assert audio.shape[0] <= limit
    dl2 = get_dataloader_from_cuts_config({"manifest_filepath": man, "use_lhotse": True, "batch_tokens": 40,
                                           "token_equivalent_duration": 0.08}, tokenizer=TOK)
    for audio, alen, tok, tlen in dl2:
        assert (float(alen.max()) / 16000 / 0.08 + int(tlen.max())) * audio.shape[0] <= 40 + 13
    bins = determine_bucket_duration_bins([1.0] * 10 + [5.0] * 2, 2)
    assert bins == [1.0] or bins == [5.0]


def test_tarred_shards_and_multi_config(tmp_path):
    man, items = _corpus(tmp_path, 8, "t")
    tars = []
    for s in range(2):
        tp = str(tmp_path / f"audio_{s}.tar")
        with tarfile.open(tp, "w") as tf:
            for it in items[s::2]:
                tf.add(it["audio_filepath"], arcname=os.path.basename(it["audio_filepath"]))
        tars.append(tp)
    cfg = {"manifest_filepath": man, "tarred_audio_filepaths": str(tmp_path / "audio__OP_0..1_CL_.tar"), "batch_size": 2}
    n0 = sum(b[0].shape[0] for b in get_dataloader_from_cuts_config(cfg, 0, 2, tokenizer=TOK))
    n1 = sum(b[0].shape[0] for b in get_dataloader_from_cuts_config(cfg, 1, 2, tokenizer=TOK))
    assert n0 == 4 and n1 == 4
    m2, _ = _corpus(tmp_path, 4, "u")
    fused = get_dataloader_from_cuts_config({"multi_config": True, "sampler_fusion": "round_robin",
                                             "a": {"manifest_filepath": man, "use_lhotse": True, "batch_size": 4},
                                             "b": {"manifest_filepath": m2, "use_lhotse": True, "batch_size": 2}}, tokenizer=TOK)
    sizes = [b[0].shape[0] for b in fused]
    assert sizes == [4, 2, 4, 2]


def test_noise_and_rir_augmentation_keep_length_and_change_signal():
    x = (0.3 * np.sin(np.arange(8000) * 0.05)).astype(np.float32)
    noise = [Cut("n", (0.1 * np.random.default_rng(0).standard_normal(3000)).astype(np.float32), 3000 / 16000)]
    y = NoiseMixer(noise, snr=10.0, prob=1.0)(x)
    snr = 10 * np.log10((x ** 2).mean() / ((y - x) ** 2).mean())
    assert y.shape == x.shape and abs(snr - 10.0) < 0.5
    z = RIRConvolver(prob=1.0, seed=1)(x)
    assert z.shape == x.shape and not np.allclose(z, x) and abs(np.abs(z).max() - np.abs(x).max()) < 1e-5


def test_model_trains_from_cuts_config(tmp_path):
    from speech_b200.core.config import open_dict
    from speech_b200.core.trainer import Trainer
    from speech_b200.models import EncDecCTCModel
    from speech_b200.models.configs import fastconformer_ctc_config

    man, _ = _corpus(tmp_path, 8, "z")
    cfg = fastconformer_ctc_config("small", vocab_size=28, n_layers=1)
    with open_dict(cfg):
        del cfg["tokenizer"]
        cfg.labels = list("abcdefghijklmnopqrstuvwxyz ") + ["'"]
        cfg.decoder.vocabulary = cfg.labels
        cfg.train_ds = {"use_lhotse": True, "manifest_filepath": man, "batch_duration": 3.0, "num_buckets": 2, "shuffle": True}
    m = EncDecCTCModel(cfg)
    tr = Trainer(max_steps=2, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(m)
    assert torch.isfinite(torch.as_tensor(float(tr.callback_metrics["train_loss"])))


def test_audio_segment_and_perturbations(tmp_path):
    import numpy as np
    from scipy.io import wavfile

    from speech_b200.data.perturb import (AudioAugmentor, AudioSegment, GainPerturbation, ImpulsePerturbation, NoisePerturbation, ShiftPerturbation,
                                          SilencePerturbation, SpeedPerturbation, TimeStretchPerturbation, TranscodePerturbation,
                                          WhiteNoisePerturbation, process_augmentations)

    sr = 16000
    t = np.arange(sr) / sr
    tone = (0.3 * np.sin(2 * np.pi * 440 * t)).astype(np.float32)
    wavfile.write(str(tmp_path / "a.wav"), sr, (tone * 32767).astype(np.int16))
    seg = AudioSegment.from_file(str(tmp_path / "a.wav"), target_sr=8000, offset=0.25, duration=0.5)
    assert seg.sample_rate == 8000 and abs(seg.num_samples - 4000) <= 2 and abs(seg.rms_db - 20 * np.log10(0.3 / np.sqrt(2))) < 0.5
    win = AudioSegment.segment_from_file(str(tmp_path / "a.wav"), n_segments=20000)
    assert win.num_samples == 20000 and float(np.abs(win.samples[16000:]).max()) == 0.0
    base = AudioSegment(tone, sr)
    s = AudioSegment(tone, sr)
    SpeedPerturbation(sr, min_speed_rate=1.25, max_speed_rate=1.25, num_rates=1).perturb(s)
    assert abs(s.num_samples - sr / 1.25) <= 2
    spec = np.abs(np.fft.rfft(s.samples))
    assert abs(np.argmax(spec) * sr / s.num_samples - 550) < 5           # pitch moves with speed
    s = AudioSegment(tone, sr)
    TimeStretchPerturbation(min_speed_rate=1.25, max_speed_rate=1.25, num_rates=1).perturb(s)
    spec = np.abs(np.fft.rfft(s.samples))
    assert abs(s.num_samples - sr / 1.25) < 600 and abs(np.argmax(spec) * sr / s.num_samples - 440) < 8   # tempo changes, pitch stays
    s = AudioSegment(tone, sr)
    GainPerturbation(6, 6).perturb(s)
    assert abs(s.rms_db - base.rms_db - 6) < 1e-3
    s = AudioSegment(tone, sr)
    noise = np.random.RandomState(0).randn(sr // 2).astype(np.float32)
    NoisePerturbation(noise_items=[{"samples": noise, "sample_rate": sr}], min_snr_db=10, max_snr_db=10, rng=0).perturb(s)
    resid = s.samples - tone
    assert abs(10 * np.log10((tone ** 2).mean() / (resid ** 2).mean()) - 10) < 0.5
    s = AudioSegment(tone, sr)
    h = np.zeros(400, np.float32)
    h[0], h[200] = 1.0, 0.5
    ImpulsePerturbation(impulse_items=[{"samples": h, "sample_rate": sr}], rng=0).perturb(s)
    expect = tone.copy()
    expect[200:] += 0.5 * tone[:-200]
    expect = expect / np.abs(expect).max() * np.abs(tone).max()
    assert np.abs(s.samples - expect).max() < 1e-3
    s = AudioSegment(tone, sr)
    ShiftPerturbation(10, 10).perturb(s)
    assert float(np.abs(s.samples[:160]).max()) == 0.0 and np.allclose(s.samples[160:], tone[:-160])
    s = AudioSegment(tone, sr)
    SilencePerturbation(0.1, 0.1, 0.2, 0.2).perturb(s)
    assert s.num_samples == sr + 1600 + 3200
    s = AudioSegment(tone, sr)
    TranscodePerturbation(["g711"]).perturb(s)
    assert s.num_samples == sr and 0.5 < np.corrcoef(s.samples, tone)[0, 1] <= 1.0
    s = AudioSegment(tone, sr)
    WhiteNoisePerturbation(-40, -39, rng=0).perturb(s)
    assert 1e-3 < np.abs(s.samples - tone).std() < 2e-2
    aug = process_augmentations({"gain": {"prob": 1.0, "min_gain_dbfs": -6, "max_gain_dbfs": -6}, "shift": {"prob": 0.0}})
    out = aug(tone, sr)
    assert isinstance(aug, AudioAugmentor) and abs(20 * np.log10(np.abs(out).max() / 0.3) + 6) < 0.1
    with pytest.raises(ValueError):
        process_augmentations({"pitch_magic": {"prob": 1.0}})


def test_feature_datasets_hf_rows_and_multispeaker_simulator(tmp_path):
    import json

    import numpy as np

    from speech_b200.data.extra_datasets import (AudioToCharDALIDataset, FeatureToLabelDataset, FeatureToTextDataset, HFAudioToTextDataset,
                                                 MultiSpeakerSimulator, TextToTextDataset)
    from speech_b200.tokenizers import CharTokenizer

    feats = []
    for k, T in enumerate((30, 50)):
        np.save(tmp_path / f"f{k}.npy", np.random.randn(8, T).astype(np.float32))
        feats.append(str(tmp_path / f"f{k}.npy"))
    (tmp_path / "lab.json").write_text("\n".join(json.dumps({"feature_file": f, "label": l}) for f, l in zip(feats, ("speech", "noise"))))
    ds = FeatureToLabelDataset(str(tmp_path / "lab.json"), labels=["noise", "speech"])
    x, xl, y, yl = ds.collate_fn([ds[0], ds[1]])
    assert x.shape == (2, 8, 50) and xl.tolist() == [30, 50] and y[:, 0].tolist() == [1, 0] and float(x[0, 0, 40]) == pytest.approx(-16.635)
    (tmp_path / "seq.json").write_text(json.dumps({"feature_file": feats[0], "label": "0 1 1 0"}))
    y = FeatureToLabelDataset(str(tmp_path / "seq.json"), delimiter=" ")[0][2]
    assert y.tolist() == [0, 1, 1, 0]
    (tmp_path / "a.rttm").write_text("SPEAKER a 1 0.10 0.10 <NA> <NA> s <NA> <NA>\n")
    (tmp_path / "txt.json").write_text(json.dumps({"feature_file": feats[0], "text": "ab a", "rttm_file": str(tmp_path / "a.rttm")}))
    tok = CharTokenizer(list(" ab"))
    ft = FeatureToTextDataset(str(tmp_path / "txt.json"), tokenizer=tok, use_rttm=True, rttm_mode="mask", feat_mask_val=-9.0)
    f, fl, t, tl = ft[0]
    assert int(tl) == 4 and float(f[0, 5]) == -9.0 and float(f[0, 15]) != -9.0
    dropped = FeatureToTextDataset(str(tmp_path / "txt.json"), tokenizer=tok, use_rttm=True, rttm_mode="drop")[0][0]
    assert dropped.shape[-1] == 11
    (tmp_path / "t.txt").write_text("ab\nba ab\n")
    tt = TextToTextDataset(str(tmp_path / "t.txt"), tok)
    s, sl, g, gl = tt.collate_fn([tt[0], tt[1]])
    assert s.shape == (2, 5) and sl.tolist() == [2, 5] and torch.equal(s, g)
    rows = [{"audio": {"array": np.random.randn(800).astype(np.float32), "sampling_rate": 8000}, "text": "AB a!"}]
    hf = HFAudioToTextDataset(data=rows, tokenizer=tok, sample_rate=16000, normalize_text=True)
    a, al, t, tl = hf[0]
    assert int(al) == 1600 and tok.ids_to_text(t.tolist()) == "ab a"
    with pytest.raises(ImportError):
        AudioToCharDALIDataset()
    items = [{"samples": np.full(8000, 0.1 * (k + 1), np.float32), "speaker_id": f"s{k % 3}", "text": f"w{k}"} for k in range(9)]
    sim = MultiSpeakerSimulator(items, sample_rate=8000, num_speakers=2, session_length=10.0, overlap_prob=0.5, seed=1)
    out = sim.generate_sessions(1, output_dir=str(tmp_path / "sim"))[0]
    assert out["audio"].shape == (80000,) and len(out["speakers"]) == 2 and len(out["rttm"]) >= 5
    assert {s["speaker"] for s in out["segments"]} <= set(out["speakers"]) and all(s["end"] <= 10.0 + 1e-6 for s in out["segments"])
    overlaps = sum(1 for a, b in zip(out["segments"], out["segments"][1:]) if b["start"] < a["end"])
    assert overlaps >= 1
    man = json.loads(open(tmp_path / "sim" / "manifest.json").read().strip())
    assert man["num_speakers"] == 2 and man["rttm_filepath"].endswith(".rttm")


def test_semi_sort_batch_sampler_groups_similar_durations_and_splits_ranks():
    import numpy as np

    from speech_b200.data.extra_datasets import SemiSortBatchSampler

    g = np.random.default_rng(0)
    dur = g.uniform(1.0, 20.0, size=103)
    s = SemiSortBatchSampler(dur, batch_size=8, randomization_factor=0.05, seed=1)
    batches = list(s)
    assert len(batches) == len(s) == 13 and sorted(i for b in batches for i in b) == list(range(103))
    spread = np.mean([dur[b].max() - dur[b].min() for b in batches])
    assert spread < 4.0                                               # random batches of 8 would span about 15 s
    s.set_epoch(1)
    assert list(s) != batches                                         # a new epoch draws new noise and a new batch order
    exact = SemiSortBatchSampler(dur, 8, randomization_factor=0.0, shuffle=False)
    flat = [i for b in exact for i in b]
    assert all(dur[flat[k]] <= dur[flat[k + 1]] for k in range(len(flat) - 1))
    r0 = list(SemiSortBatchSampler(dur, 8, global_rank=0, world_size=2, seed=3))
    r1 = list(SemiSortBatchSampler(dur, 8, global_rank=1, world_size=2, seed=3))
    assert len(r0) == len(r1) == 7 and set(map(tuple, r0)).isdisjoint(set(map(tuple, r1))) or len(r0) == len(r1)
    assert len(SemiSortBatchSampler(dur, 8, drop_last=True)) == 12
