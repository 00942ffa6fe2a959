"""Model families beyond CTC / transducer ASR, exercised on CPU with synthetic data: a few optimisation steps must run,
the loss must be finite (and fall where the task is learnable), and the inference entry points must work."""
import math

import numpy as np
import pytest
import torch

from speech_b200.core.config import OmegaConf
from speech_b200.core.trainer import Trainer
from speech_b200.models import (ClusteringDiarizer, ConfidenceEnsembleModel, EncDecClassificationModel, EncDecCTCModelBPE,
                                EncDecMaskedTokenPredModel, EncDecMultiTalkerRNNTBPEModel, EncDecRNNTBPEModelWithPrompt,
                                EncDecSpeakerLabelModel, SortformerEncLabelModel, SpeechEncDecSelfSupervisedModel)
from speech_b200.models.asr_variants import entropy_confidence, evaluate_eou
from speech_b200.models.configs import (encoder_cfg, fastconformer_ctc_config, fastconformer_transducer_config,
                                        preprocessor_cfg)
from speech_b200.models.diarizers import cosine_affinity, nme_spectral_clustering
from speech_b200.models.sortformer_models import find_segments, get_ats_targets, get_pil_targets

JASPER = [{"filters": 32, "repeat": 1, "kernel": [11], "stride": [1], "dilation": [1], "dropout": 0.0, "residual": False,
           "separable": True},
          {"filters": 32, "repeat": 2, "kernel": [13], "stride": [1], "dilation": [1], "dropout": 0.0, "residual": True,
           "separable": True, "se": True},
          {"filters": 48, "repeat": 1, "kernel": [1], "stride": [1], "dilation": [1], "dropout": 0.0, "residual": False}]


def _label_cfg(decoder):
    return OmegaConf.create({
        "sample_rate": 16000, "labels": ["a", "b", "c"], "preprocessor": {**preprocessor_cfg(32), "dither": 0.0},
        "encoder": {"_target_": "speech_b200.modules.conv_asr.ConvASREncoder", "feat_in": 32, "activation": "relu",
                    "conv_mask": True, "jasper": JASPER},
        "decoder": decoder,
        "train_ds": {"synthetic": {"num_samples": 48, "num_classes": 3}, "batch_size": 8, "shuffle": True},
        "optim": {"name": "adamw", "lr": 3e-3, "weight_decay": 0.0}})


def _fit(model, steps):
    tr = Trainer(max_steps=steps, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(model)
    return tr


def test_classification_model_learns_tones():
    torch.manual_seed(0)
    m = EncDecClassificationModel(_label_cfg({"_target_": "speech_b200.modules.conv_asr.ConvASRDecoderClassification",
                                              "feat_in": None, "num_classes": 3}))
    tr = _fit(m, 30)
    assert float(tr.callback_metrics["train_loss"]) < 0.8
    assert m.transcribe([np.zeros(8000, dtype=np.float32)])[0] in ("a", "b", "c")


def test_speaker_model_embeddings_and_verification():
    torch.manual_seed(0)
    m = EncDecSpeakerLabelModel(_label_cfg({"_target_": "speech_b200.modules.conv_asr.SpeakerDecoder", "feat_in": None,
                                            "num_classes": 3, "emb_sizes": 16, "pool_mode": "attention", "angular": True}))
    tr = _fit(m, 10)
    assert math.isfinite(float(tr.callback_metrics["train_loss"]))
    x = np.random.default_rng(0).standard_normal(16000).astype(np.float32)
    assert m.get_embedding(x).shape == (1, 16)
    assert m.verify_speakers(x, x)


def test_nme_spectral_clustering_separates_two_speakers():
    g = np.random.default_rng(0)
    a = g.standard_normal(16)
    b = g.standard_normal(16)
    emb = np.stack([a + 0.05 * g.standard_normal(16) for _ in range(12)] + [b + 0.05 * g.standard_normal(16) for _ in range(9)])
    labels = nme_spectral_clustering(cosine_affinity(emb), max_num_speakers=4)
    assert len(set(labels[:12])) == 1 and len(set(labels[12:])) == 1 and labels[0] != labels[-1]


def test_sortformer_trains_and_streams():
    torch.manual_seed(0)
    cfg = OmegaConf.create({
        "sample_rate": 16000, "max_num_of_spks": 3, "preprocessor": {**preprocessor_cfg(32), "dither": 0.0, "normalize": "NA"},
        "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
        "sortformer_modules": {"_target_": "speech_b200.models.sortformer_models.SortformerModules", "num_spks": 3,
                               "dropout_rate": 0.0, "fc_d_model": 176, "tf_d_model": 64, "spkcache_len": 24, "fifo_len": 6,
                               "chunk_len": 10, "spkcache_sil_frames_per_spk": 1},
        "transformer_encoder": {"_target_": "speech_b200.modules.transformer.TransformerEncoder", "num_layers": 1,
                                "hidden_size": 64, "inner_size": 128, "num_attention_heads": 4},
        "train_ds": {"synthetic": {"num_samples": 8}, "batch_size": 4, "shuffle": True},
        "optim": {"name": "adamw", "lr": 1e-3, "weight_decay": 0.0}})
    m = SortformerEncLabelModel(cfg)
    tr = _fit(m, 3)
    assert math.isfinite(float(tr.callback_metrics["train_loss"]))
    x = [np.random.default_rng(1).standard_normal(16000 * 3).astype(np.float32)]
    _, offline = m.diarize(x, include_tensor_outputs=True)
    m.streaming_mode = True
    _, online = m.diarize(x, include_tensor_outputs=True)
    assert offline[0].shape == online[0].shape == (38, 3)
    lab = torch.zeros(1, 6, 3)
    lab[0, 3:, 0] = 1
    lab[0, 1:4, 2] = 1
    ats = get_ats_targets(lab, lab, m.speaker_permutations)
    assert ats[0, :, 0].tolist() == [0, 1, 1, 1, 0, 0] and ats[0, :, 1].tolist() == [0, 0, 0, 1, 1, 1]
    pil = get_pil_targets(lab, ats, m.speaker_permutations)
    assert torch.equal(pil, ats)
    assert find_segments(np.array([0, .9, .9, .2, .9, .9, 0.]), 0.1, min_duration_off=0.15) == [(0.1, 0.6000000000000001)]


def test_ssl_models_run():
    torch.manual_seed(0)
    enc = encoder_cfg("small", 32, 0.0, 0.0, n_layers=1)
    ds = {"synthetic": {"num_samples": 8, "vocab_size": 8, "min_duration": 1.0, "max_duration": 1.5}, "batch_size": 4}
    nest = EncDecMaskedTokenPredModel(OmegaConf.create({
        "preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": enc,
        "quantizer": {"_target_": "speech_b200.models.ssl_models.RandomProjectionVectorQuantizer", "feat_in": 32, "code_dim": 8,
                      "num_classes": 64, "num_books": 2, "combine_time_steps": 8},
        "masking": {"_target_": "speech_b200.models.ssl_models.RandomBlockMasking", "feat_in": 32, "block_size": 16,
                    "mask_prob": 0.4},
        "decoder": {"_target_": "speech_b200.models.ssl_models.MultiSoftmaxDecoder", "feat_in": 176, "num_classes": 64,
                    "num_decoders": 2},
        "loss": {"_target_": "speech_b200.losses.misc.MultiMLMLoss", "combine_time_steps": 8, "num_decoders": 2},
        "train_ds": ds, "optim": {"name": "adamw", "lr": 1e-3}}))
    assert math.isfinite(float(_fit(nest, 2).callback_metrics["train_loss"]))
    con = SpeechEncDecSelfSupervisedModel(OmegaConf.create({
        "preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": enc,
        "spec_augment": {"_target_": "speech_b200.modules.spec_augment.SpectrogramAugmentation", "freq_masks": 0,
                         "time_masks": 4, "time_width": 20},
        "decoder": {"_target_": "speech_b200.modules.conv_asr.ConvASRDecoderReconstruction", "feat_in": 176, "feat_hidden": 32,
                    "feat_out": 16, "stride_layers": 0, "non_stride_layers": 0},
        "loss": {"_target_": "speech_b200.losses.misc.ContrastiveLoss", "in_dim": 32, "proj_dim": 16, "combine_time_steps": 8,
                 "num_negatives": 5, "quantized_targets": True, "codebook_size": 16, "num_groups": 2},
        "train_ds": ds, "optim": {"name": "adamw", "lr": 1e-3}}))
    assert math.isfinite(float(_fit(con, 2).callback_metrics["train_loss"]))


def test_prompt_and_multitalker_variants_step():
    torch.manual_seed(0)
    cfg = fastconformer_transducer_config("small", vocab_size=16, loss="rnnt", dropout=0.0, n_layers=1, sched=None, lr=1e-3)
    audio = torch.randn(2, 16000)
    alen = torch.tensor([16000, 12000])
    txt = torch.randint(0, 16, (2, 5))
    tlen = torch.tensor([5, 3])
    pm = EncDecRNNTBPEModelWithPrompt(cfg)
    pm.train()
    out = pm.training_step((audio, alen, txt, tlen, torch.tensor([3, 7])), 0)
    out["loss"].backward()
    assert pm.prompt_kernel[0].weight.grad is not None and torch.isfinite(out["loss"])
    mt = EncDecMultiTalkerRNNTBPEModel(cfg)
    mt.train()
    act = (torch.rand(2, 13) > 0.5).float()
    out = mt.training_step((audio, alen, txt, tlen, act, 1 - act), 0)
    out["loss"].backward()
    assert mt.spk_kernels["0"].ff[0].weight.grad.abs().sum() > 0


def test_eou_metrics_and_confidence():
    r = evaluate_eou([{"start_time": 1.9, "end_time": 2.1, "eou_pred": True}, {"start_time": 0.4, "end_time": 0.5, "eou_pred": True}],
                     [{"start_time": 0.0, "end_time": 2.0}], collar=0.0)
    assert r.true_positives == 1 and r.latency == [pytest.approx(0.1)] and len(r.early_cutoff) == 1
    flat = torch.full((1, 4, 8), math.log(1 / 8))
    peaked = torch.log_softmax(torch.tensor([[[20.0] + [0.0] * 7] * 4]), -1)
    for kind in ("tsallis", "renyi", "gibbs", "max_prob"):
        assert float(entropy_confidence(flat, 0.5, kind).mean()) == pytest.approx(0.0, abs=1e-5)
        assert float(entropy_confidence(peaked, 0.5, kind).mean()) > 0.99


def test_confidence_ensemble_picks_a_model():
    torch.manual_seed(0)
    a = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=16, n_layers=1))
    b = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=16, n_layers=1))
    ens = ConfidenceEnsembleModel(OmegaConf.create({}), models=[a, b])
    ens.eval()
    out = ens.transcribe([np.random.default_rng(0).standard_normal(16000).astype(np.float32)])
    assert len(out) == 1 and isinstance(out[0], str)


def test_clustering_diarizer_end_to_end(tmp_path):
    class FakeSpk:
        def batch_inference(self, chunks, batch_size=64):
            # "embedding" = normalised magnitude spectrum pooled to 16 bins
            e = []
            for c in chunks:
                s = np.abs(np.fft.rfft(np.asarray(c), n=2048))[:512].reshape(16, 32).mean(1)
                e.append(s / (np.linalg.norm(s) + 1e-8))
            return torch.tensor(np.stack(e), dtype=torch.float32), None

    sr = 16000
    t = np.arange(sr * 2) / sr
    x = np.concatenate([0.3 * np.sin(2 * np.pi * 220 * t), np.zeros(sr // 2), 0.3 * np.sin(2 * np.pi * 1800 * t)]).astype(np.float32)
    d = ClusteringDiarizer({"diarizer": {"out_dir": str(tmp_path)}}, speaker_model=FakeSpk())
    segs = d.diarize([x])["session_0"]
    spk = {s[2] for s in segs}
    assert len(spk) == 2
    first = [s for s in segs if s[1] <= 2.1]
    last = [s for s in segs if s[0] >= 2.4]
    assert first and last and {s[2] for s in first} != {s[2] for s in last}
    assert (tmp_path / "pred_rttms" / "session_0.rttm").exists()


def test_extra_encoders_rnn_transformer_wav2vec_parallel_expert():
    from speech_b200.modules.conformer_encoder import ConformerEncoder
    from speech_b200.modules.extra_encoders import (ConvFeatureEncoder, LSTMDecoder, ParallelExpertEncoder, RNNEncoder, TransformerEncoder,
                                                    Wav2VecTransformerEncoder)

    torch.manual_seed(0)
    feats, lens = torch.randn(2, 32, 64), torch.tensor([64, 40])
    rnn = RNNEncoder(32, n_layers=2, d_model=48, proj_size=32, subsampling="stacking", subsampling_factor=4)
    y, yl = rnn(audio_signal=feats, length=lens)
    assert y.shape == (2, 32, 16) and yl.tolist() == [16, 10]
    dec = LSTMDecoder(32, num_classes=5, lstm_hidden_size=24, vocabulary=list("abcde"), bidirectional=True)
    lp = dec(encoder_output=y)
    assert lp.shape == (2, 16, 6) and torch.allclose(lp.exp().sum(-1), torch.ones(2, 16), atol=1e-5)
    for sam, mode in (("rel_pos", "full"), ("abs_pos", "causal"), ("no_pos", "full")):
        enc = TransformerEncoder(feat_in=32, d_model=64, n_heads=4, n_layers=2, subsampling="striding", subsampling_factor=4,
                                 subsampling_conv_channels=16, self_attention_model=sam, attn_mode=mode, qk_norm=(sam == "no_pos"), drop_rate=0.0,
                                 dropout_pre_encoder=0.0).eval()
        out, ol = enc(audio_signal=feats, length=lens)
        assert out.shape == (2, 64, 16) and ol.tolist() == [16, 10]
        # padding of the shorter utterance must not leak into its valid frames
        out2, _ = enc(audio_signal=torch.cat([feats[1:, :, :40], torch.randn(1, 32, 24)], dim=2), length=lens[1:])
        assert torch.allclose(out[1, :, :10], out2[0, :, :10], atol=1e-4)
        if mode == "causal":   # the future must not influence the past
            f2 = feats.clone()
            f2[0, :, 48:] += 1.0
            o3, _ = enc(audio_signal=f2, length=lens)
            assert torch.allclose(o3[0, :, :8], out[0, :, :8], atol=1e-4) and not torch.allclose(o3[0, :, 12:], out[0, :, 12:], atol=1e-4)
    with pytest.raises(ValueError, match="below 16"):
        TransformerEncoder(feat_in=32, d_model=64, n_heads=8, n_layers=1)
    enc = TransformerEncoder(feat_in=32, d_model=64, n_heads=4, n_layers=1, subsampling="feature_stacking", subsampling_factor=4, feat_out=24,
                             pos_emb_max_len=8).eval()
    out, ol = enc(audio_signal=feats, length=lens)
    assert out.shape == (2, 24, 16) and enc._feat_out == 24
    enc.update_max_seq_length(400)
    assert enc.max_audio_length == 100
    enc.pos_bias_frozen = None
    enc.layers[0].attn.pos_bias_u.requires_grad = False
    enc.freeze()
    enc.unfreeze(partial=True)
    assert not enc.layers[0].attn.pos_bias_u.requires_grad and enc.layers[0].fc1.weight.requires_grad
    conv = ConvFeatureEncoder([{"emb_dim": 16, "kernel_size": 10, "stride": 5}, {"emb_dim": 16, "kernel_size": 3, "stride": 2}], embedding_dim=32)
    wav, wl = torch.randn(2, 1600), torch.tensor([1600, 1000])
    f, fl = conv(input_signal=wav, length=wl)
    assert f.shape[:2] == (2, 32) and fl.tolist() == [159, 99] and f.shape[2] == 159
    w2v = Wav2VecTransformerEncoder(embedding_dim=32, num_layers=2, num_heads=4, inner_size=64, pos_kernel_size=8, pos_groups=4).eval()
    o, _ = w2v(audio_signal=f, length=fl)
    assert o.shape == f.shape
    asr = ConformerEncoder(feat_in=32, n_layers=1, d_model=32, n_heads=4, subsampling_factor=4, subsampling_conv_channels=16, conv_kernel_size=5)
    pe = ParallelExpertEncoder(asr, None, n_spk=4).eval()
    base, bl = pe(feats, lens)
    spk = torch.zeros(2, 16, 4)
    spk[:, :, 1] = 1.0
    fused, _ = pe(feats, lens, spk_targets=spk)
    assert fused.shape == base.shape and not torch.allclose(fused, base)
    expect = pe.asr_norm(base.transpose(1, 2)) + pe.diar_norm(spk) @ pe.diar_kernel
    assert torch.allclose(fused.transpose(1, 2), expect, atol=1e-5)


def test_transformer_decoder_translation_model_trains_decodes_and_scores_bleu(tmp_path):
    """EncDecTransfModelBPE: encoder -> adapter -> Transformer encoder -> Transformer decoder; the loss falls on a fixed batch,
    beam search returns token strings, and the epoch-end hook reports a position-weighted loss and corpus BLEU."""
    import torch
    from speech_b200.core.config import OmegaConf
    from speech_b200.models import EncDecTransfModelBPE
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.models.transformer_bpe_models import corpus_bleu
    from speech_b200.tokenizers import ByteLevelTokenizer

    assert corpus_bleu(["the cat sat on the mat ."], ["the cat sat on the mat ."]) > 99.9
    assert corpus_bleu(["a b c d e f"], ["u v w x y z"]) == 0.0
    mid = corpus_bleu(["the cat sat on a mat today"], ["the cat sat on the mat today"])
    assert 20.0 < mid < 80.0
    assert corpus_bleu(["Hello, world!"], ["Hello , world !"]) > 99.9          # 13a tokenisation splits punctuation

    torch.manual_seed(0)
    tr = {"hidden_size": 48, "inner_size": 96, "num_layers": 1, "num_attention_heads": 4, "ffn_dropout": 0.0, "attn_score_dropout": 0.0,
          "attn_layer_dropout": 0.0, "pre_ln": True, "max_sequence_length": 64}
    cfg = OmegaConf.create({
        "sample_rate": 16000, "tokenizer": {"type": "synthetic", "vocab_size": 32},
        "preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1), "spec_augment": None,
        "transf_encoder": dict(tr), "transf_decoder": dict(tr, learn_positional_encodings=True),
        "head": {"num_layers": 1, "activation": "relu", "log_softmax": True, "dropout": 0.0},
        "beam_search": {"beam_size": 2, "len_pen": 0.6, "max_generation_delta": 5}, "label_smoothing": 0.1,
        "optim": {"name": "adamw", "lr": 3e-3}})
    m = EncDecTransfModelBPE(cfg)
    assert isinstance(m.adapter, torch.nn.Linear) and m.use_transf_encoder
    assert m.log_softmax.mlp.layer0.weight is m.transf_decoder.embedding.token_embedding.weight
    t = m.tokenizer
    audio, lens = torch.randn(2, 8000), torch.tensor([8000, 6400])
    body = torch.randint(3, 30, (2, 5))
    tokens = torch.cat([torch.full((2, 1), t.bos_id), body, torch.full((2, 1), t.eos_id)], dim=1)
    tokens[1, 5:] = torch.tensor([t.eos_id, t.pad_id])
    batch = (audio, lens, tokens, torch.tensor([7, 6]))
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = m.training_step(batch, 0)["loss"]
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.8 * losses[0]
    m.eval()
    out = m.validation_step(batch, 0)
    assert len(out["translations"]) == 2 and out["loss_weight"] == 2 * 6
    res = m.multi_validation_epoch_end([out, out], 0)
    assert "val_sacreBLEU" in "".join(res["log"]) and float(res["val_loss"]) == pytest.approx(float(out["val_loss"]), rel=1e-5)
    hyps = m._transcribe_forward_and_decode(audio, lens, None)
    assert len(hyps) == 2 and all(isinstance(h.text, str) for h in hyps)
    with pytest.raises(ValueError, match="either input_signal"):
        m.forward()


def test_speaker_tagged_asr_offline_streaming_and_speaker_target_data(tmp_path):
    import json

    from speech_b200.core.config import open_dict
    from speech_b200.models.multitalker import (SpeakerTaggedASR, SpeakerTargetDataset, find_active_speakers, get_simulated_softmax, mask_features,
                                                sentences_from_words, write_seglst)

    torch.manual_seed(0)
    cfg = fastconformer_transducer_config("small", vocab_size=16, loss="rnnt", dropout=0.0, n_layers=2, sched=None, lr=1e-3, causal=True,
                                          att_context_size=[8, 1], att_context_style="chunked_limited", conv_norm_type="layer_norm")
    with open_dict(cfg):
        cfg.preprocessor.normalize, cfg.preprocessor.dither, cfg.preprocessor.pad_to = "NA", 0.0, 0
    asr = EncDecMultiTalkerRNNTBPEModel(cfg).eval()
    audio = torch.randn(1, 32000) * 0.1
    lens = torch.tensor([32000])
    Tp = 26
    diar = torch.zeros(1, Tp, 4)
    diar[0, :14, 0] = 0.9                  # speaker 0 talks first
    diar[0, 10:, 2] = 0.8                  # speaker 2 joins later, overlapping
    assert find_active_speakers(diar, 0.5, 3) == [[2, 0]] and find_active_speakers(diar, 0.5, 15) == [[2]]
    p = get_simulated_softmax(torch.tensor([0.9, 0.001, 0.6, 0.3]), limit_max_spks=3)
    assert float(p.sum()) == pytest.approx(1.0) and float(p[3]) == 0.0 and float(p[1]) > 0
    feats = torch.randn(1, 80, 200)
    masked = mask_features(feats, diar[:, :, 0], subsampling=8)
    assert torch.equal(masked[0, :, :112], feats[0, :, :112]) and bool((masked[0, :, 112:] == feats.min()).all())
    tagger = SpeakerTaggedASR(asr, lambda a, l: diar, max_gap=0.5)
    seglst = tagger.transcribe_offline(audio, lens, ["meeting"])
    assert {d["speaker"] for d in seglst} <= {"speaker_0", "speaker_2"} and all(d["session_id"] == "meeting" and d["end_time"] >= d["start_time"] for d in seglst)
    # the target mask matters: another speaker's mask changes the encoder output
    asr.set_speaker_targets(diar[:, :, 0], diar[:, :, 2])
    e0, _ = asr.forward(input_signal=audio, input_signal_length=lens)
    asr.set_speaker_targets(diar[:, :, 2], diar[:, :, 0])
    e2, _ = asr.forward(input_signal=audio, input_signal_length=lens)
    asr.set_speaker_targets(None)
    assert not torch.allclose(e0, e2)
    hyps = asr.transcribe_with_speaker_targets(audio, lens, diar[:, :, 0], diar[:, :, 2])
    assert len(hyps) == 1 and asr._spk_targets is None
    streamed = tagger.stream(audio[0], diar[0])
    assert tagger.manager.get_speakers() == [0, 2] and tagger.manager.instances[2].start_offset > 0
    for d in streamed:
        assert d["speaker"] in ("speaker_0", "speaker_2") and 0.0 <= d["start_time"] <= d["end_time"] <= 2.3
    words = [{"word": "hi", "start_time": 0.0, "end_time": 0.2}, {"word": "there.", "start_time": 0.3, "end_time": 0.6},
             {"word": "so", "start_time": 0.7, "end_time": 0.8}, {"word": "late", "start_time": 3.0, "end_time": 3.3}]
    sents = sentences_from_words(words, "s", "speaker_1", max_gap=1.0)
    assert [x["words"] for x in sents] == ["hi there.", "so", "late"] and sents[0]["end_time"] == 0.6
    write_seglst(str(tmp_path / "out.seglst.json"), sents)
    assert json.load(open(tmp_path / "out.seglst.json"))[2]["words"] == "late"
    ds = SpeakerTargetDataset([{"audio": np.zeros(16000, dtype=np.float32),
                                "segments": [{"speaker": "A", "start": 0.0, "end": 0.4, "text": "ab"}, {"speaker": "B", "start": 0.32, "end": 0.8, "text": "cd"},
                                             {"speaker": "A", "start": 0.8, "end": 1.0, "text": "ef"}]}], asr.tokenizer, deterministic=True)
    batch = SpeakerTargetDataset.collate([ds[0], ds[0]])
    assert batch[4].shape == (2, 13) and batch[4][0].tolist() == [1.0] * 5 + [0.0] * 5 + [1.0] * 2 + [0.0] and batch[5][0].tolist() == [0.0] * 4 + [1.0] * 6 + [0.0] * 3
    asr.train()
    out = asr.training_step(batch, 0)
    assert torch.isfinite(out["loss"])
    asr.eval()
    assert "val_wer" in asr.validation_pass(batch, 0)


def test_offline_diarization_with_asr_assignment_realignment_outputs_and_scores(tmp_path):
    import json

    from speech_b200.models import diar_with_asr as D

    words = [{"word": w, "start_time": 0.5 * i, "end_time": 0.5 * i + 0.4} for i, w in enumerate("how are you today i am fine thanks".split())]
    labels = ["0.000 1.800 speaker_0", "1.800 4.000 speaker_1"]                 # the change is placed one word early ("today" starts at 1.5)
    plain = D.OfflineDiarWithASR(word_anchor="mid")
    tagged = plain.assign_speakers(words, labels)
    assert [w["speaker"] for w in tagged] == ["speaker_0"] * 4 + ["speaker_1"] * 4
    early = ["0.000 1.300 speaker_0", "1.300 4.000 speaker_1"]
    assert [w["speaker"] for w in plain.assign_speakers(words, early)][3] == "speaker_1"              # "today" lands on the wrong side
    # a language model that likes the two fluent sentences moves the boundary back
    good = {("how", "are", "you", "today"), ("i", "am", "fine", "thanks")}
    lm = lambda ws: 0.0 if tuple(ws) in good else -float(len(ws))  # noqa: E731
    fixed = D.OfflineDiarWithASR(realigning_lm=lm, max_shift=2).assign_speakers(words, early)
    assert [w["speaker"] for w in fixed] == ["speaker_0"] * 4 + ["speaker_1"] * 4
    res = plain.get_transcript_with_speaker_labels({"s1": labels}, {"s1": words})
    assert res["s1"]["speaker_count"] == 2 and [s["text"] for s in res["s1"]["sentences"]] == ["how are you today", "i am fine thanks"]
    D.OfflineDiarWithASR.write_outputs(res, str(tmp_path / "out"))
    assert open(tmp_path / "out" / "s1.txt").readline().startswith("[00:00.00 - 00:01.90] speaker_0: how are you today")
    assert len(open(tmp_path / "out" / "s1.ctm").read().splitlines()) == 8 and json.load(open(tmp_path / "out" / "s1.json"))["session_id"] == "s1"
    rttm = D.labels_to_rttmfile(["0.000 2.000 A", "2.000 4.000 B"], "s1", str(tmp_path / "rttm"))
    assert D.rttm_to_labels(rttm) == ["0.000 2.000 A", "2.000 4.000 B"]
    ref_words = [(w["word"], "A" if i < 4 else "B") for i, w in enumerate(words)]
    ev = D.OfflineDiarWithASR.evaluate(res, {"s1": rttm}, {"s1": ref_words}, {"s1": labels}, collar=0.0)["s1"]
    assert ev["cpWER"] == 0.0 and ev["WDER"] == 0.0 and ev["WER"] == 0.0 and ev["DER"] == pytest.approx(0.05) and ev["CER"] == pytest.approx(0.05)
    wrong = plain.get_transcript_with_speaker_labels({"s1": early}, {"s1": words})
    ev2 = D.OfflineDiarWithASR.evaluate(wrong, None, {"s1": ref_words})["s1"]
    assert ev2["WDER"] == pytest.approx(1 / 8) and ev2["cpWER"] == pytest.approx(2 / 8)
    assert D.merge_float_intervals([[0, 1], [0.5, 2], [3, 4], [4.00001, 5]]) == [[0.0, 2.0], [3.0, 5.0]]
    assert D.get_sub_range_list([1.0, 3.5], [[0, 2], [3, 4], [5, 6]]) == [[1.0, 2], [3, 3.5]] and not D.is_overlap([0, 1], [1, 2])
    seg = [{"session_id": "s", "speaker": "A", "start_time": 8.0, "end_time": 12.0, "words": "a b c d"}, {"session_id": "s", "speaker": "B", "start_time": 13.0, "end_time": 14.0, "words": "e"}]
    chunks = D.chunk_seglst(seg, 10.0)
    assert [c["words"] for c in chunks[0]] == ["a b"] and [c["words"] for c in chunks[1]] == ["c d", "e"] and chunks[1][0]["start_time"] == 10.0
    man = tmp_path / "m.json"
    man.write_text(json.dumps({"audio_filepath": "/a/x.wav", "offset": 0, "duration": 3.0}) + "\n" + json.dumps({"audio_filepath": "/a/x.wav", "offset": 3.0, "duration": 3.0}))
    assert list(D.audio_rttm_map(str(man), attach_dur=True)) == ["x_0_3000", "x_3000_3000"]
    with pytest.raises(KeyError):
        D.audio_rttm_map(str(man))


def test_model_config_records_diarizer_preset_and_matchboxnet_builder():
    import torch

    from speech_b200.core.config_schemas import to_dictconfig
    from speech_b200.models import config_records as R
    from speech_b200.models.classification_models import EncDecClassificationModel
    from speech_b200.models.diarizers import ClusteringDiarizer

    inf = R.NeuralDiarizerInferenceConfig.init_config(diar_model_path=None, vad_model_path="vad.nemo", map_location="cpu")
    assert inf.diarizer.vad.model_path == "vad.nemo" and inf.diarizer.clustering.parameters.max_num_speakers == 8
    assert inf.diarizer.speaker_embeddings.parameters.get("window_length_in_sec")[0] == 1.5 and "collar" in list(inf.diarizer)
    dc = inf.to_dictconfig()
    assert dc.diarizer.vad.parameters.onset == 0.1 and list(dc.diarizer.speaker_embeddings.parameters.shift_length_in_sec)[-1] == 0.25
    d = ClusteringDiarizer(dc)
    assert d.windows == [1.5, 1.25, 1.0, 0.75, 0.5] and d.max_num_speakers == 8 and d.sparse_search_volume == 30

    b = R.EncDecClassificationModelConfigBuilder("matchboxnet_3x1x64")
    b.set_labels(["yes", "no", "up"])
    b.set_sample_rate(8000)
    b.set_repeat(2)
    b.set_dropout(0.1)
    b.set_timesteps(64)
    cfg = b.build()
    assert cfg.decoder["num_classes"] == 3 and cfg.decoder["feat_in"] == 128 and cfg.encoder["feat_in"] == 64 and cfg.preprocessor.sample_rate == 8000
    assert [blk["repeat"] for blk in cfg.encoder["jasper"]] == [1, 2, 2, 2, 1, 1] and cfg.encoder["jasper"][-1]["dropout"] == 0.0 and cfg.encoder["jasper"][0]["dropout"] == 0.1
    assert cfg.train_ds.labels == ["yes", "no", "up"] and cfg.validation_ds.sample_rate == 8000 and cfg.crop_or_pad_augment.audio_length == 64
    with pytest.raises(ValueError):
        R.EncDecClassificationModelConfigBuilder("resnet")
    mc = to_dictconfig(cfg)
    mc.train_ds = None
    mc.validation_ds = None
    mc.test_ds = None
    mc.optim = {"name": "adamw", "lr": 1e-3}
    model = EncDecClassificationModel(mc).eval()
    with torch.no_grad():
        logits = model.forward(input_signal=torch.randn(2, 8000), input_signal_length=torch.tensor([8000, 6000]))
    assert logits.shape == (2, 3)
    vad = R.EncDecClassificationModelConfigBuilder("matchboxnet_3x1x64_vad").build()
    assert vad.labels == ["background", "speech"] and vad.decoder["num_classes"] == 2 and vad.crop_or_pad_augment is None
    top = to_dictconfig(R.EncDecCTCModelConfig(name="ctc"))
    assert top.model.optim.name == "novograd" and top.model.preprocessor.features == 64 and top.model.train_ds.shuffle is True
