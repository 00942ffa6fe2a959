"""TTS collection on CPU: FSQ round trip, codec training step, transformer KV cache, MoE routing, alignment prior / loss,
MagpieTTS training and autoregressive inference."""
import math

import pytest
import torch

from speech_b200.core.config import OmegaConf
from speech_b200.core.trainer import Trainer
from speech_b200.tokenizers import CharTokenizer
from speech_b200.tts.audio_codec import AudioCodecModel, FiniteScalarQuantizer, GroupFiniteScalarQuantizer
from speech_b200.tts.magpietts import ForwardSumLoss, MagpieTTSModel, beta_binomial_prior
from speech_b200.tts.transformer_2501 import MoERouter, Transformer

CODEC_CFG = {"sample_rate": 8000, "train_discriminator": True,
             "audio_encoder": {"encoded_dim": 8, "down_sample_rates": [4, 4, 4], "base_channels": 8},
             "vector_quantizer": {"num_groups": 2, "num_levels_per_group": [4, 4, 3, 3]},
             "audio_decoder": {"input_dim": 8, "up_sample_rates": [4, 4, 4], "base_channels": 32, "resblock_kernel_sizes": [3]},
             "discriminator": {"periods": [2, 3], "stft_resolutions": [[256, 64, 256]]},
             "mel_loss": {"n_mels": 20, "n_fft": 256, "hop": 64, "win": 256},
             "train_ds": {"synthetic": {"num_samples": 8, "min_duration": 0.3, "max_duration": 0.5, "sample_rate": 8000}, "batch_size": 4},
             "optim": {"lr": 1e-3}}


def test_fsq_indices_round_trip():
    torch.manual_seed(0)
    q = FiniteScalarQuantizer([8, 5, 5, 5])
    x = torch.randn(2, 4, 7) * 2
    lens = torch.tensor([7, 4])
    deq, idx = q(x, lens)
    assert idx.shape == (1, 2, 7) and int(idx.max()) < q.codebook_size == 1000
    assert torch.allclose(q.decode(idx, lens), deq, atol=1e-6)
    assert float(deq[1, :, 4:].abs().sum()) == 0.0
    g = GroupFiniteScalarQuantizer(2, [4, 4, 3])
    d2, i2 = g(torch.randn(2, 6, 5), torch.tensor([5, 5]))
    assert i2.shape == (2, 2, 5) and torch.allclose(g.decode(i2, torch.tensor([5, 5])), d2, atol=1e-6)
    x.requires_grad_(True)
    q(x, lens)[0].sum().backward()
    assert x.grad.abs().sum() > 0                    # straight-through gradient


def test_codec_trains_and_tokens_round_trip():
    torch.manual_seed(0)
    m = AudioCodecModel(OmegaConf.create(CODEC_CFG))
    m.configure_optimizers()
    audio = torch.randn(2, 2048) * 0.1
    lens = torch.tensor([2048, 1500])
    out = m.training_step((audio, lens), 0)
    out["loss"].backward()
    assert math.isfinite(float(out["loss"]))
    m.eval()
    tokens, tlen = m.encode(audio, lens)
    assert tokens.shape[:2] == (2, 2) and tlen.tolist() == [32, 24]
    rec, rlen = m.decode(tokens, tlen)
    assert rec.shape[0] == 2 and rlen.tolist() == [2048, 1536]


def test_transformer_kv_cache_matches_full_pass_and_moe_balances():
    torch.manual_seed(0)
    t = Transformer(n_layers=2, d_model=32, d_ffn=64, sa_n_heads=4, kernel_size=1, has_xattn=True, xa_d_memory=16, xa_n_heads=2,
                    is_causal=True, use_learnable_pos_emb=True, max_length_causal_mask=64).eval()
    x, cond = torch.randn(2, 6, 32), torch.randn(2, 5, 16)
    xm, cm = torch.ones(2, 6, dtype=torch.bool), torch.ones(2, 5, dtype=torch.bool)
    full = t(x, xm, cond=cond, cond_mask=cm)["output"]
    cache = t.new_cache()
    steps = [t(x[:, i:i + 1], xm[:, i:i + 1], cond=cond, cond_mask=cm, cache=cache, position_offset=i)["output"] for i in range(6)]
    assert torch.allclose(torch.cat(steps, 1), full, atol=1e-4)
    r = MoERouter(16, num_experts=4, top_k=2)
    w, e, aux = r(torch.randn(64, 16))
    assert w.shape == (64, 2) and torch.allclose(w.sum(-1), torch.ones(64), atol=1e-5)
    assert float(aux["load_balancing_loss"]) >= 0.99            # equals 1 for perfectly uniform routing, larger otherwise
    moe = Transformer(n_layers=1, d_model=16, d_ffn=32, sa_n_heads=2, use_moe=True, num_experts=3, top_k_experts=1)
    y = moe(torch.randn(2, 5, 16), torch.ones(2, 5, dtype=torch.bool))["output"]
    assert y.shape == (2, 5, 16) and "load_balancing_loss" in moe.moe_aux_losses()


def test_alignment_prior_and_forward_sum_loss():
    p = beta_binomial_prior(5, 12)
    assert p.shape == (12, 5) and torch.allclose(p.sum(1), torch.ones(12), atol=1e-4)
    assert int(p[0].argmax()) == 0 and int(p[-1].argmax()) == 4          # diagonal band
    loss = ForwardSumLoss()
    diag = torch.full((1, 12, 5), -8.0)
    for t in range(12):
        diag[0, t, min(4, t * 5 // 12)] = 0.0
    anti = diag.flip(2)
    tl, al = torch.tensor([5]), torch.tensor([12])
    assert float(loss(diag, tl, al)) < float(loss(anti, tl, al))


def test_magpie_trains_and_synthesises():
    torch.manual_seed(0)
    codec = AudioCodecModel(OmegaConf.create({**CODEC_CFG, "train_discriminator": False}))
    tok = CharTokenizer(list("abcdefgh "))
    tf = dict(n_layers=1, d_model=32, d_ffn=64, sa_n_heads=2, kernel_size=1, p_dropout=0.0)
    cfg = OmegaConf.create({
        "embedding_dim": 32, "frame_stacking_factor": 2, "num_special_audio_tokens": 4,
        "encoder": dict(tf, is_causal=False), "decoder": dict(tf, has_xattn=True, xa_d_memory=32, xa_n_heads=1, is_causal=True,
                                                             use_learnable_pos_emb=True, max_length_causal_mask=256),
        "local_transformer_type": "autoregressive", "local_transformer_n_layers": 1, "local_transformer_hidden_dim": 32,
        "alignment_loss_scale": 0.1, "alignment_decoder_loss_layers": [0], "prior_scaling_factor": 0.5, "cfg_unconditional_prob": 0.1,
        "train_ds": {"synthetic": {"num_samples": 8}, "batch_size": 4}, "optim": {"name": "adamw", "lr": 2e-3, "weight_decay": 0.0}})
    m = MagpieTTSModel(cfg, codec=codec, tokenizer=tok)
    assert not any(n.startswith("_codec") for n, _ in m.named_parameters())
    tr = Trainer(max_steps=3, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(m)
    assert math.isfinite(float(tr.callback_metrics["train_loss"])) and "train_alignment_loss" in tr.callback_metrics
    audio, alen = m.do_tts("abc", max_decoder_steps=6, use_cfg=True)
    assert audio.shape[0] == 1 and 0 < int(alen[0]) <= audio.shape[1]
    long = m.generate_speech("ab. cd! ef?", max_chars_per_chunk=4, max_decoder_steps=3)
    assert long.numel() > 0


def test_classic_tts_g2p_alignment_fastpitch_vocoder_aligner():
    from speech_b200.tts.classic import (AlignerModel, DictG2p, FastPitchModel, HifiGanModel, PhonemeTokenizer, binarize_attention,
                                         regulate_len)

    g2p = DictG2p({"hello": [["HH", "AH0", "L", "OW1"]], "read": [["R", "IY1", "D"], ["R", "EH1", "D"]]})
    assert g2p("Hello, read xyz") == ["HH", "AH0", "L", "OW1", ",", " ", "r", "e", "a", "d", " ", "x", "y", "z"]
    tok = PhonemeTokenizer(g2p)
    ids = tok.text_to_ids("hello world")
    assert tok.ids_to_tokens(ids)[:4] == ["HH", "AH0", "L", "OW1"] and tok.oov not in ids
    # monotonic alignment search: a diagonal-dominant soft attention gives a staircase that covers every text position once
    T, N = 9, 3
    soft = torch.full((1, T, N), 0.05)
    for t in range(T):
        soft[0, t, t * N // T] = 0.9
    hard = binarize_attention(soft, torch.tensor([N]), torch.tensor([T]))
    assert hard.sum(2).tolist() == [[1.0] * T] and hard.sum(1).tolist() == [[3.0, 3.0, 3.0]]
    out, lens = regulate_len(torch.tensor([[2.0, 0.0, 3.0]]), torch.arange(3.0).view(1, 3, 1))
    assert lens.tolist() == [5] and out[0, :, 0].tolist() == [0.0, 0.0, 2.0, 2.0, 2.0]
    torch.manual_seed(0)
    cfg = OmegaConf.create({"n_symbols": tok.vocab_size, "symbols_embedding_dim": 32, "d_inner": 64, "encoder_layers": 1, "decoder_layers": 1,
                            "n_mel_channels": 20, "sample_rate": 8000, "n_fft": 256, "hop_length": 64, "win_length": 256, "bin_loss_warmup_epochs": 0})
    fp = FastPitchModel(cfg, tokenizer=tok)
    text = torch.tensor([ids + [0] * 2, tok.text_to_ids("hello") + [0] * (len(ids) - 2)])
    text_len = torch.tensor([len(ids), 4])
    t = torch.arange(4000) / 8000.0
    audio = torch.stack([torch.sin(2 * math.pi * 150 * t), torch.sin(2 * math.pi * 220 * t)]) * 0.5
    f0 = FastPitchModel.estimate_pitch(audio, 64, 8000)
    assert abs(float(f0[0, 10:40].median()) - 150) < 8 and abs(float(f0[1, 10:40].median()) - 220) < 12
    loss = fp.training_step((text, text_len, audio, torch.tensor([4000, 3000])), 0)["loss"]
    loss.backward()
    assert math.isfinite(float(loss)) and fp.duration_predictor.fc.weight.grad is not None
    mel = fp.generate_spectrogram(fp.parse("hello"))
    assert mel.shape[:2] == (1, 20)
    voc = HifiGanModel(OmegaConf.create({"sample_rate": 8000, "generator": {"input_dim": 20, "up_sample_rates": [4, 4, 4], "base_channels": 32,
                                                                          "resblock_kernel_sizes": [3]},
                                         "discriminator": {"periods": [2, 3], "stft_resolutions": [[256, 64, 256]]},
                                         "mel": {"n_fft": 256, "hop": 64, "win": 256}}))
    voc.configure_optimizers()
    wav = voc.convert_spectrogram_to_audio(torch.randn(1, 20, 10))
    assert wav.shape == (1, 640)
    vl = voc.training_step((audio[:, :2048], torch.tensor([2048, 2048])), 0)["loss"]
    assert math.isfinite(float(vl))
    al = AlignerModel(OmegaConf.create({"n_symbols": tok.vocab_size, "symbols_embedding_dim": 16, "n_mel_channels": 80, "sample_rate": 8000}), tokenizer=tok)
    l2 = al.training_step((text, text_len, audio, torch.tensor([4000, 3000])), 0)["loss"]
    l2.backward()
    assert math.isfinite(float(l2))


def test_preference_losses_and_grpo_math():
    from speech_b200.tts.preference import grpo_advantages, grpo_loss, preference_loss, sequence_logprob

    torch.manual_seed(0)
    logits = torch.randn(2, 5, 3, 7)
    tgt = torch.randint(0, 7, (2, 5, 3))
    mask = torch.tensor([[1.0, 1, 1, 1, 1], [1, 1, 1, 0, 0]])
    lp = sequence_logprob(logits, tgt, mask)
    ref = torch.log_softmax(logits, -1).gather(-1, tgt.unsqueeze(-1)).squeeze(-1).sum(-1)
    assert torch.allclose(lp[1], ref[1, :3].sum()) and torch.allclose(lp[0], ref[0].sum())
    pc, pr, rc, rr = torch.tensor([-10.0]), torch.tensor([-12.0]), torch.tensor([-11.0]), torch.tensor([-11.0])
    loss, c, r = preference_loss(pc, pr, rc, rr, beta=0.5, loss_type="dpo")
    assert torch.allclose(loss, -torch.nn.functional.logsigmoid(torch.tensor(0.5 * 2.0))) and float(c) > float(r)
    assert float(preference_loss(pc, pr, rc, rr, beta=0.5, loss_type="ipo")[0]) == pytest.approx((2.0 - 1.0) ** 2)
    assert float(preference_loss(pc, pr, rc, rr, 0.5, "rpo_sq", torch.tensor([1.0]), torch.tensor([0.0]))[0]) == pytest.approx(0.0)
    with pytest.raises(NotImplementedError):
        preference_loss(pc, pr, rc, rr, loss_type="xyz")
    adv = grpo_advantages(torch.tensor([[1.0, 2.0, 3.0], [5.0, 5.0, 5.0]]))
    assert torch.allclose(adv[0].mean(), torch.tensor(0.0), atol=1e-6) and float(adv[1].abs().max()) == 0.0 and float(adv[0, 2]) > 1.0
    new = torch.tensor([-5.0, -6.0], requires_grad=True)
    l = grpo_loss(new, new.detach(), torch.tensor([1.0, -1.0]), ref_logp=torch.tensor([-5.5, -6.0]), kl_beta=0.1, lengths=torch.tensor([5, 5]))
    l.backward()
    assert new.grad[0] < 0 < new.grad[1]          # raise the likelihood of the above-average sample, lower the other
