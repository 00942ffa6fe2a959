"""TTS collection on CPU: FSQ round trip, codec training step, transformer KV cache, MoE routing, alignment prior / loss,
MagpieTTS training and autoregressive inference."""
import math
import os
import re

import numpy as np

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


def test_mamba2_chunked_equals_recurrence_and_easy_magpie_trains_and_generates():
    import math

    from speech_b200.core.config import OmegaConf
    from speech_b200.tts.easy_magpie import EasyMagpieTTSModel, Mamba2Block, NemotronHDecoder

    torch.manual_seed(0)
    blk = Mamba2Block(32, d_state=8, head_dim=8, n_groups=2, chunk_size=5).eval()
    u = torch.randn(2, 13, 32)
    full = blk(u)
    cache = {}
    first = blk(u[:, :4], cache)                                     # chunked prefill fills the cache ...
    steps = [blk(u[:, t:t + 1], cache) for t in range(4, 13)]        # ... and the O(1) recurrence continues from it
    inc = torch.cat([first] + steps, dim=1)
    assert torch.allclose(full, inc, atol=1e-4), float((full - inc).abs().max())
    one = Mamba2Block(32, d_state=8, head_dim=8, n_groups=2, chunk_size=64).eval()
    one.load_state_dict(blk.state_dict())
    assert torch.allclose(one(u), full, atol=1e-4)                   # the chunk length does not change the result
    tiny = dict(vocab_size=40, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8)
    from speech_b200.speechlm.llm import LLMConfig

    dec = NemotronHDecoder(LLMConfig(**tiny), "M-*-M", {"d_state": 8, "head_dim": 8}).eval()
    x = torch.randn(2, 9, 32)
    ref = dec(x)
    c = dec.new_cache()
    got = torch.cat([dec(x[:, :5], c)] + [dec(x[:, t:t + 1], c) for t in range(5, 9)], dim=1)
    assert torch.allclose(ref, got, atol=1e-4)
    for backbone in ("transformer", "nemotron_h"):
        cfg = OmegaConf.create({"backbone_type": backbone, "backbone": tiny, "hybrid_pattern": "M*-", "mamba": {"d_state": 8, "head_dim": 8},
                                "num_codebooks": 3, "codebook_size": 12, "optim": {"name": "adamw", "lr": 1e-3}})
        m = EasyMagpieTTSModel(cfg)
        batch = {"text": torch.randint(0, 40, (2, 7)), "text_len": torch.tensor([7, 5]), "codes": torch.randint(0, 12, (2, 3, 10)),
                 "codes_len": torch.tensor([10, 6])}
        loss = m.training_step(batch, 0)["loss"]
        loss.backward()
        assert math.isfinite(float(loss)) and m.heads[2].weight.grad is not None and m.text_emb.weight.grad is not None
        # the EOS frame is the last target of every utterance
        _, tgt, mask = m(batch["text"], batch["text_len"], batch["codes"], batch["codes_len"])
        assert int(tgt[1, 6, 0]) == m.audio_eos_id and bool(mask[1, 6]) and not bool(mask[1, 7])
        codes, lens = m.infer_batch(batch["text"], max_steps=6, generator=torch.Generator().manual_seed(0))
        assert codes.shape[:2] == (2, 3) and codes.shape[2] <= 6 and (codes.numel() == 0 or int(codes.max()) < 12) and lens.shape == (2,)
        # greedy decoding with caches equals teacher forcing on its own output
        g, gl = m.infer_batch(batch["text"][:1], max_steps=4, temperature=0.0)
        if g.shape[2] > 1:
            lg, _, _ = m(batch["text"][:1], torch.tensor([7]), g, torch.tensor([g.shape[2]]))
            lg = lg[0, : g.shape[2]].clone()
            lg[..., m.audio_bos_id] = float("-inf")
            lg[:, 1:, m.audio_eos_id] = float("-inf")
            assert torch.equal(lg.argmax(-1).t(), g[0])


def _magpie_cfg(local="none", **extra):
    tf = dict(n_layers=1, d_model=32, d_ffn=64, sa_n_heads=2, kernel_size=1, p_dropout=0.0)
    return OmegaConf.create({
        "embedding_dim": 32, "frame_stacking_factor": 1, "num_special_audio_tokens": 4,
        "encoder": dict(tf, is_causal=False), "decoder": dict(tf, has_xattn=True, xa_d_memory=32, xa_n_heads=1, is_causal=True,
                                                             use_learnable_pos_emb=True, max_length_causal_mask=256),
        "local_transformer_type": local, "local_transformer_n_layers": 1, "local_transformer_hidden_dim": 32,
        "train_ds": {"synthetic": {"num_samples": 8}, "batch_size": 4}, "optim": {"name": "adamw", "lr": 2e-3, "weight_decay": 0.0}, **extra})


def test_magpie_maskgit_local_transformer_and_cfg_distillation():
    from speech_b200.tts.cfg_distillation import MagpieTTSModelOnlineCFGDistillation, distillation_kl, guided_logits

    torch.manual_seed(0)
    codec = AudioCodecModel(OmegaConf.create({**CODEC_CFG, "train_discriminator": False}))
    tok = CharTokenizer(list("abcdefgh "))
    m = MagpieTTSModel(_magpie_cfg("maskgit"), codec=codec, tokenizer=tok)
    tr = Trainer(max_steps=2, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(m)
    assert math.isfinite(float(tr.callback_metrics["train_local_transformer_loss"]))
    h = torch.randn(5, 32)
    codes = m._local_maskgit(h, temperature=0.7, topk=10, n_steps=3)
    C = len(m.audio_embeddings)
    assert codes.shape == (5, C) and int(codes.max()) <= m.audio_eos_id          # every codebook decided, no mask / BOS left
    audio, alen = m.do_tts("abc", max_decoder_steps=4)
    assert audio.shape[0] == 1 and int(alen[0]) > 0
    # guided logits and the KL objective
    c, u = torch.randn(2, 3, 4, 7), torch.randn(2, 3, 4, 7)
    assert torch.allclose(guided_logits(c, u, 1.0), c, atol=1e-5) and torch.allclose(guided_logits(c, u, 0.0), u)
    mask = torch.ones(2, 3, dtype=torch.bool)
    assert float(distillation_kl(c, c, mask)) < 1e-6 and float(distillation_kl(c, u, mask)) > 0
    teacher = MagpieTTSModel(_magpie_cfg(), codec=codec, tokenizer=tok)
    stu = MagpieTTSModelOnlineCFGDistillation(_magpie_cfg(cfg_scale_range=[1.0, 3.0], ce_weight=0.1), codec=codec, tokenizer=tok, teacher=teacher)
    assert not any(n.startswith("_teacher") for n, _ in stu.named_parameters())
    tr = Trainer(max_steps=2, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(stu)
    assert math.isfinite(float(tr.callback_metrics["train_distillation_loss"])) and 1.0 <= float(tr.callback_metrics["train_cfg_scale"]) <= 3.0
    assert all(p.grad is None for p in teacher.parameters())
    out = stu.infer_batch(torch.tensor([[1, 2, 3]]), torch.tensor([3]), cfg_scale=2.0, max_decoder_steps=3)
    assert out[0].shape[0] == 1


def test_tts_eval_metrics_frechet_similarity_rtf_harness():
    from speech_b200.tts.eval_metrics import (FrechetCodecDistance, MosPredictorWrapper, RTFMetrics, evaluate_tts, frechet_distance,
                                              intelligibility, speaker_similarity)

    g = torch.Generator().manual_seed(0)
    mu, cov = torch.zeros(3), torch.eye(3)
    assert frechet_distance(mu, cov, mu, cov) < 1e-9
    # closed form for axis-aligned Gaussians: |dmu|^2 + sum (s1 - s2)^2
    d = frechet_distance(torch.tensor([1.0, 0, 0]), torch.diag(torch.tensor([4.0, 1, 1])), mu, cov)
    assert abs(d - (1.0 + 1.0)) < 1e-6
    fcd = FrechetCodecDistance()
    real = torch.randn(4000, 6, generator=g)
    fcd.update(real_latents=real[:2000], fake_latents=real[2000:])
    near = fcd.compute()
    far = FrechetCodecDistance()
    far.update(real_latents=real[:2000], fake_latents=real[2000:] * 2 + 1)
    assert near < 0.1 < far.compute()
    emb = lambda a, l: torch.stack([a.mean(-1), a.std(-1)], dim=-1)  # noqa: E731
    x = torch.randn(2, 100, generator=g) + 1
    assert torch.allclose(speaker_similarity(emb, x, None, x, None), torch.ones(2), atol=1e-6)
    sc = intelligibility(lambda auds: ["Hello, world", "good bye"], [None, None], ["hello world", "good day"])
    assert abs(sc["wer"] - 0.25) < 1e-9 and sc["cer"] > 0
    r = RTFMetrics(100)
    r.timed(lambda: None)
    r.add_audio(250)
    assert r.compute()["audio_seconds"] == 2.5
    mos = MosPredictorWrapper(lambda x, sr: x.abs().mean(-1), 100, batch_size=2)
    assert len(mos([torch.ones(5), torch.ones(9), torch.zeros(3)])) == 3

    class _Fake:
        def do_tts(self, text, **kw):
            n = 50 * len(text)
            return torch.ones(1, n), torch.tensor([n])

    res = evaluate_tts(_Fake(), [{"text": "ab", "audio": torch.ones(80)}, {"text": "abcd"}], 100, transcribe=lambda a: ["ab", "abcd"],
                       speaker_embed=emb, mos=mos)
    assert res["wer"] == 0.0 and res["utterances"] == 2 and abs(res["audio_seconds"] - 3.0) < 1e-9 and "speaker_similarity" in res and "mos" in res


def test_ssl_disentangler_heads_and_losses():
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.tts.classic import SSLDisentangler

    torch.manual_seed(0)
    cfg = OmegaConf.create({"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
                            "encoder_dim": 176, "content_emb_dim": 24, "speaker_emb_dim": 16, "num_phonemes": 11, "num_speakers": 3,
                            "optim": {"name": "adamw", "lr": 1e-3}})
    m = SSLDisentangler(cfg)
    audio, alen = torch.randn(2, 16000), torch.tensor([16000, 11000])
    logits, content, spk_logits, spk, elen = m(audio, alen)
    assert logits.shape[-1] == 12 and content.shape[-1] == 24 and spk_logits.shape == (2, 3) and spk.shape == (2, 16)
    assert torch.allclose(spk.norm(dim=-1), torch.ones(2), atol=1e-5)
    # per-utterance normalisation of the content embedding: zero mean over the valid frames, nothing beyond them
    n1 = int(elen[1])
    assert float(content[1, :n1].detach().mean(0).abs().max()) < 1e-4 and float(content[1, n1:].detach().abs().sum()) == 0
    out = m.training_step((audio, alen, torch.randint(0, 11, (2, 5)), torch.tensor([5, 3]), torch.tensor([0, 2])), 0)
    out["loss"].backward()
    assert math.isfinite(float(out["loss"])) and m.speaker_out.weight.grad is not None and m.content_out.weight.grad is not None


def test_code_token_models_train_through_the_trainer_on_synthetic_codes():
    from speech_b200.speechlm.ear_tts import DuplexEARTTS
    from speech_b200.tts.easy_magpie import EasyMagpieTTSModel

    torch.manual_seed(0)
    tiny = dict(vocab_size=40, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2, head_dim=8)
    ds = {"synthetic": {"num_samples": 8}, "batch_size": 4}
    em = EasyMagpieTTSModel(OmegaConf.create({"backbone_type": "nemotron_h", "backbone": tiny, "hybrid_pattern": "M*-", "mamba": {"d_state": 8, "head_dim": 8},
                                              "num_codebooks": 2, "codebook_size": 12, "train_ds": ds, "validation_ds": ds,
                                              "optim": {"name": "adamw", "lr": 1e-3}}))
    tr = Trainer(max_steps=3, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(em)
    assert math.isfinite(float(tr.callback_metrics["train_loss"]))
    ear = DuplexEARTTS(OmegaConf.create({"tts": {"backbone": tiny, "num_quantizers": 3, "codebook_size": 16, "latent_size": 8, "num_predictions": 4,
                                                 "low_rank": 4}, "train_ds": ds, "optim": {"name": "adamw", "lr": 1e-3}}))
    tr = Trainer(max_steps=3, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False)
    tr.fit(ear)
    assert math.isfinite(float(tr.callback_metrics["train_loss"]))


@pytest.mark.parametrize("model_type", ["multi_encoder_context_tts", "decoder_context_tts", "decoder_ce"])
def test_magpie_voice_context_attention_prior_and_long_form_state(model_type):
    from speech_b200.tts.magpietts import LongFormState, split_text_for_tts

    torch.manual_seed(0)
    codec = AudioCodecModel(OmegaConf.create({**CODEC_CFG, "train_discriminator": False}))
    tok = CharTokenizer(list("abcdefgh .,"))
    tf = dict(n_layers=1, d_model=32, d_ffn=64, sa_n_heads=2, kernel_size=1, p_dropout=0.0)
    m = MagpieTTSModel(_magpie_cfg(model_type=model_type, context_encoder=dict(tf, is_causal=False), alignment_decoder_loss_layers=[0],
                                   prior_scaling_factor=0.5, alignment_loss_scale=0.1, context_duration_max=0.1), codec=codec, tokenizer=tok)
    assert hasattr(m, "context_encoder") == (model_type != "decoder_context_tts")
    text = torch.randint(0, 8, (2, 6))
    tl = torch.tensor([6, 4])
    audio, al = torch.randn(2, 1600) * 0.1, torch.tensor([1600, 1280])
    ctx_audio, cl = torch.randn(2, 960) * 0.1, torch.tensor([960, 640])
    m.train()
    loss, logs = m._loss((text, tl, audio, al, ctx_audio, cl))
    loss.backward()
    assert math.isfinite(float(loss)) and "alignment_loss" in logs
    if model_type != "decoder_context_tts":
        assert next(m.context_encoder.parameters()).grad is not None
    # the context changes the prediction; cross-attention returned to the caller covers text positions only
    m.eval()
    codes, n = m.stack_codes(*m.audio_to_codes(audio, al))
    cc, cn = m.stack_codes(*m.audio_to_codes(ctx_audio, cl))
    with torch.no_grad():
        lg_a, attn, _, _ = m(text, tl, codes, n, context_codes=cc, context_codes_len=cn)
        lg_b, _, _, _ = m(text, tl, codes, n, context_codes=cc.flip(-1), context_codes_len=cn)
        lg_0, _, _, _ = m(text, tl, codes, n)
    assert lg_a.shape == lg_0.shape and not torch.allclose(lg_a, lg_b)
    m.train()
    with torch.no_grad():
        attn = m(text, tl, codes, n, context_codes=cc, context_codes_len=cn)[1]
    m.eval()
    assert attn[0].shape[-2:] == (codes.shape[-1] - 1, 6)
    out = m.infer_batch(text, tl, max_decoder_steps=6, context_codes=cc, context_codes_len=cn, attention_prior_strength=4.0,
                        attention_prior_window=2, return_attention=True)
    assert out[2].shape[0] == 2 and out[4].shape[0] == 2 and out[4].shape[2] == 6
    # long-form: chunks share the voice context, state is kept on the model
    chunks = split_text_for_tts("abc def. gh ab, cd ef gh ab cd. a b.", 12)
    assert all(len(c) <= 12 for c in chunks) and " ".join(chunks).replace(" ", "") == "abcdef.ghab,cdefghabcd.ab."
    wav = m.generate_speech("abc def. gh ab. cd ef.", max_chars_per_chunk=8, max_decoder_steps=3, crossfade_ms=1.0)
    st = m.last_long_form_state
    assert isinstance(st, LongFormState) and st.chunks_done == 3 and st.context_codes is not None and wav.numel() > 0
    wav2 = m.generate_speech("abc. def.", max_chars_per_chunk=5, max_decoder_steps=3, context_audio=ctx_audio[0])
    assert m.last_long_form_state.context_codes.shape[-1] == int(cn[0]) and wav2.numel() > 0


def test_causal_codec_decoder_streams_chunk_by_chunk_to_the_same_audio():
    from speech_b200.tts.audio_codec_extra import CausalHiFiGANDecoder

    torch.manual_seed(0)
    dec = CausalHiFiGANDecoder(input_dim=8, up_sample_rates=(4, 2), base_channels=16, resblock_kernel_sizes=(3,), resblock_dilation_sizes=(1, 3)).eval()
    z = torch.randn(2, 8, 12)
    with torch.no_grad():
        full, lens = dec(z, torch.tensor([12, 12]))
        state, chunks = None, []
        for a, b in ((0, 5), (5, 6), (6, 12)):
            y, state = dec.decode_stream(z[:, :, a:b], state)
            chunks.append(y)
        # causality: changing a later latent frame leaves earlier samples alone
        z2 = z.clone()
        z2[:, :, 8:] += 1.0
        full2, _ = dec(z2, torch.tensor([12, 12]))
    assert full.shape == (2, 96) and lens.tolist() == [96, 96]
    assert torch.allclose(torch.cat(chunks, dim=-1), full, atol=1e-5)
    assert torch.allclose(full2[:, : 8 * 8], full[:, : 8 * 8], atol=1e-6) and not torch.allclose(full2[:, 64:], full[:, 64:])


def test_codec_discriminators_and_losses():
    from speech_b200.tts.audio_codec_extra import (
        DiscriminatorHingedLoss, DiscriminatorSquaredLoss, GeneratorHingedLoss, GeneratorSquaredLoss, MMDLoss, MultiBandDiscriminatorSTFT,
        MultiResolutionDiscriminatorSTFT, MultiResolutionMelLoss, RelativeFeatureMatchingLoss, ResNetSpeakerEncoder, SISDRLoss, SLMDiscriminator,
        TimeDomainLoss,
    )

    torch.manual_seed(0)
    real, gen = torch.randn(2, 4000), torch.randn(2, 4000)
    mrd = MultiResolutionDiscriminatorSTFT(resolutions=((128, 32, 128), (256, 64, 256)), ch=4)
    sr, sg, fr, fg = mrd(real, gen)
    assert len(sr) == 2 and sr[0].dim() == 2 and len(fr[0]) == 5 * 4 + 1
    assert MultiBandDiscriminatorSTFT((128, 32, 128), ch=4)(real)[0].shape[0] == 2
    # a stand-in foundation model: 3 "layers" of framed audio
    extract = lambda a: torch.stack([a.unfold(-1, 16, 160)] * 3, dim=1)  # noqa: E731
    slm = SLMDiscriminator(extract, slm_hidden=16, slm_layers=3, initial_channel=4, input_sr=22050, slm_sr=16000)
    s_r, s_g, f_r, f_g = slm(real, gen)
    assert s_r[0].shape == s_g[0].shape and len(f_r[0]) == 3
    for gl, dl, fake in ((GeneratorHingedLoss(), DiscriminatorHingedLoss(), -1.0), (GeneratorSquaredLoss(), DiscriminatorSquaredLoss(), 0.0)):
        assert float(dl([torch.full((2, 3), 1.0)], [torch.full((2, 3), fake)])) == 0.0             # a perfect discriminator
        assert float(dl([torch.full((2, 3), 0.0)], [torch.full((2, 3), 0.5)])) > 0.0
        assert float(gl([torch.full((2, 3), 1.0)])) == 0.0 and float(gl([torch.full((2, 3), 0.0)])) == 1.0
    assert float(RelativeFeatureMatchingLoss()(fr, fr)) == 0.0 and float(RelativeFeatureMatchingLoss()(fr, fg)) > 0
    lens = torch.tensor([4000, 3000])
    assert float(TimeDomainLoss()(real, real, lens)) == 0.0
    mel = MultiResolutionMelLoss(16000, resolutions=((64, 16), (256, 64)), mel_dims=(10, 40))
    assert float(mel(real, real, lens)) == 0.0 and float(mel(real, gen, lens)) > 0
    # SI-SDR ignores scale and is clipped; noise lowers it
    sd = SISDRLoss(clip_max=30.0)
    assert float(sd(real, 3.0 * real)) == pytest.approx(-30.0, abs=1e-3)
    assert float(sd(real, real + 0.1 * gen, lens)) == pytest.approx(-20.0, abs=1.5)
    mmd = MMDLoss()
    a, b = torch.randn(200, 6), torch.randn(200, 6)
    assert abs(float(mmd(a, b))) < 0.02 < float(mmd(a, b + 2.0))
    emb = ResNetSpeakerEncoder(n_mels=16, channels=(4, 8), proj_dim=12).eval()(torch.randn(2, 8000))
    assert emb.shape == (2, 12) and torch.allclose(emb.norm(dim=-1), torch.ones(2), atol=1e-5)


def test_codec_index_converter_round_trips_between_group_layouts():
    from speech_b200.tts.audio_codec import GroupFiniteScalarQuantizer
    from speech_b200.tts.audio_codec_extra import VectorQuantizerIndexConverter

    old, new = GroupFiniteScalarQuantizer(4, [4, 4]), GroupFiniteScalarQuantizer(2, [4, 4, 4, 4])
    conv = VectorQuantizerIndexConverter(old, new)
    lens = torch.tensor([7, 5])
    z = torch.randn(2, 8, 7)
    deq_old, idx_old = old(z, lens)
    idx_new = conv.convert_original_to_new(idx_old)
    assert idx_new.shape == (2, 2, 7) and int(idx_new.max()) < 256
    # the new layout decodes to the very same latent values, and the way back restores the indices
    assert torch.allclose(new.decode(idx_new, lens), deq_old, atol=1e-6)
    assert torch.equal(conv.convert_new_to_original(idx_new), idx_old)
    with pytest.raises(ValueError):
        VectorQuantizerIndexConverter(old, GroupFiniteScalarQuantizer(2, [8, 4, 4, 2]))


def test_audio_codec_model_with_causal_decoder_slm_discriminator_and_hinged_losses():
    torch.manual_seed(0)
    cfg = OmegaConf.create({
        "sample_rate": 16000, "mel_loss": {"n_mels": 20, "n_fft": 256, "hop": 64, "win": 256}, "gan_loss": "hinged", "feature_loss_type": "relative", "time_domain_loss_scale": 1.0, "si_sdr_loss_scale": 0.1,
        "audio_encoder": {"down_sample_rates": [4, 2], "base_channels": 8, "encoded_dim": 8},
        "vector_quantizer": {"num_groups": 2, "num_levels_per_group": [4, 4, 4, 4]},
        "audio_decoder": {"causal": True, "input_dim": 8, "up_sample_rates": [2, 4], "base_channels": 16, "resblock_kernel_sizes": [3], "resblock_dilation_sizes": [1, 3]},
        "discriminator": {"periods": [2], "stft_resolutions": [], "multiband_stft_resolutions": [[128, 32, 128]]},
    })
    m = AudioCodecModel(cfg)
    m.add_slm_discriminator(lambda a: torch.stack([a.unfold(-1, 16, 160)] * 2, dim=1), slm_hidden=16, slm_layers=2, initial_channel=4, slm_sr=16000)
    m.configure_optimizers()
    assert any(n.startswith("discriminator.slm.") for n, _ in m.named_parameters())
    audio, lens = torch.randn(2, 3200), torch.tensor([3200, 2400])
    out = m.training_step((audio, lens), 0)
    out["loss"].backward()
    assert torch.isfinite(out["loss"])
    # tokens -> audio in two chunks equals the one-shot decode
    m.eval()
    toks, tl = m.encode(audio, torch.tensor([3200, 3200]))
    full, _ = m.decode(toks, tl)
    a, st = m.decode_stream(toks[..., :150])
    b, st = m.decode_stream(toks[..., 150:], st)
    assert torch.allclose(torch.cat([a, b], -1), full, atol=1e-5)


def test_ipa_pinyin_and_kana_g2p(tmp_path):
    from speech_b200.tts.g2p import ChineseG2p, IpaG2p, JapaneseG2p, phoneme_error_rate

    p = tmp_path / "ipa.txt"
    p.write_text("HELLO\thəˈloʊ\nWORLD\tˈwɝld\nREAD\tˈɹid, ˈɹɛd\nCAT\tˈkæt\nWELL\tˈwɛl\nKNOWN\tˈnoʊn\nT͡ʃIP\tt͡ʃɪp\n", encoding="utf-8")
    g = IpaG2p(str(p), heteronyms=["read"], grapheme_prefix="#")
    assert g("hello world") == ["h", "ə", "ˈ", "l", "o", "ʊ", " ", "ˈ", "w", "ɝ", "l", "d"]
    assert g("read")[:2] == ["#R", "#E"]                               # heteronym: left as (prefixed) graphemes
    assert g("cat's cats")[:5] == ["ˈ", "k", "æ", "t", "s"] and g("cat's cats")[-1] == "s"
    assert g("well-known") == ["ˈ", "w", "ɛ", "l", "-", "ˈ", "n", "o", "ʊ", "n"]
    assert g("xyzzy!") == ["#X", "#Y", "#Z", "#Z", "#Y", "!"]          # unknown word spelled, punctuation kept
    assert IpaG2p.split_ipa("t͡ʃɪːp") == ["t͡ʃ", "ɪː", "p"]
    nostress = IpaG2p(str(p), use_stresses=False)
    assert "ˈ" not in nostress("hello")
    amb = IpaG2p({"read": ["ɹid", "ɹɛd"]}, ignore_ambiguous_words=False, grapheme_case="lower")
    assert amb("read") == ["ɹ", "i", "d"]
    amb.replace_symbols(["ɹ", "ɛ", "d"])
    assert amb("read") == ["ɹ", "ɛ", "d"]
    zh = ChineseG2p({"你好": "ni3 hao3", "世": "shi4", "界": "jie4"})
    assert zh("你好世界 OK") == ["n", "i", "#3", "h", "ao", "#3", "sh", "i", "#4", "j", "ie", "#4", " ", "O", "K"]
    ja = JapaneseG2p()
    assert ja("きょう") == ["k", "j", "o", "ɯ"] and ja("ガッコー") == ["g", "a", "k", "k", "oː"] and ja("シャ") == ["ɕ", "a"]
    with pytest.raises(ValueError):
        ja("今日")
    assert JapaneseG2p(kana_reader=lambda s: "キョウ")("今日") == ["k", "j", "o", "ɯ"]
    assert phoneme_error_rate([["a", "b"]], [["a", "c", "d"]]) == pytest.approx(2 / 3)


@pytest.mark.parametrize("kind", ["ctc", "seq2seq"])
def test_neural_g2p_models_learn_a_toy_lexicon(kind, tmp_path):
    import json

    from speech_b200.tts.g2p import CTCG2PModel, Seq2SeqG2PModel

    torch.manual_seed(0)
    lex = [("cat", "k æ t"), ("tack", "t æ k"), ("act", "æ k t"), ("box", "b ɑ k s"), ("tax", "t æ k s"), ("cab", "k æ b")]
    phon = sorted({p for _, s in lex for p in s.split()})
    cfg = OmegaConf.create({"phonemes": phon, "d_model": 32, "n_layers": 1, "n_heads": 2, "upsample": 2,
                            "train_ds": {"examples": [[g, p] for g, p in lex], "batch_size": 6, "shuffle": False}})
    m = (CTCG2PModel if kind == "ctc" else Seq2SeqG2PModel)(cfg)
    opt = torch.optim.Adam(m.parameters(), 5e-3)
    batch = next(iter(m._train_dl))
    first = None
    for _ in range(150):
        opt.zero_grad()
        loss = m.training_step(batch, 0)["loss"]
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss)
    assert float(loss) < 0.2 * first
    assert m.predict(["cat", "box"]) == [["k", "æ", "t"], ["b", "ɑ", "k", "s"]]       # "box": more phonemes than letters
    assert float(m.validation_step(batch, 0)["val_per"]) == 0.0
    src, dst = tmp_path / "in.json", tmp_path / "out.json"
    src.write_text("\n".join(json.dumps({"text_graphemes": g}) for g, _ in lex[:3]), encoding="utf-8")
    preds = m.convert_graphemes_to_phonemes(str(src), str(dst))
    assert preds == [s for _, s in lex[:3]] and json.loads(dst.read_text(encoding="utf-8").splitlines()[1])["pred_text"] == "t æ k"


def test_tts_data_stack_vocoder_magpie_featurizers_processors_trimming(tmp_path):
    import json

    import numpy as np

    from speech_b200.data.audio_to_text import save_wav
    from speech_b200.tts.data_extra import (BetaBinomialInterpolator, ChunkedTTSInferenceDataset, EnergyAudioTrimmer, EnergyFeaturizer, FeatureScaler,
                                            LanguageThresholds, LogCompression, MagpieTTSDataset, MagpieTTSDatasetDPO, MeanVarianceNormalization,
                                            MeanVarianceSpeakerNormalization, MelSpectrogramFeaturizer, PitchFeaturizer, VadAudioTrimmer, VocoderDataset,
                                            normalize_volume)

    sr = 16000
    t = np.arange(sr) / sr
    rows = {"a": [], "b": []}
    for name, n, f0 in (("a", 4, 200.0), ("b", 1, 330.0)):
        for k in range(n):
            p = tmp_path / f"{name}{k}.wav"
            save_wav(str(p), (0.3 * np.sin(2 * np.pi * f0 * t)).astype(np.float32), sr)
            rows[name].append({"audio_filepath": p.name, "duration": 1.0, "text": f"hello {name} {k}. " * 2, "speaker": name, "language": "en",
                               "reward": float(k % 2 == 0)})
        (tmp_path / f"{name}.json").write_text("\n".join(json.dumps(r) for r in rows[name]))
    meta = {n: {"manifest_path": str(tmp_path / f"{n}.json"), "audio_dir": str(tmp_path), "sample_weight": w} for n, w in (("a", 1.0), ("b", 1.0))}
    voc = VocoderDataset(meta, sr, weighted_sampling_steps_per_epoch=50, n_samples=4000, resample_rates=[8000], volume_norm=True,
                         feature_processors={"scale": FeatureScaler("audio", div_value=2.0)})
    sampler = voc.get_sampler(batch_size=4)
    drawn = [voc.samples[i]["dataset_name"] for i in sampler]
    assert len(drawn) == 200 and 0.35 < drawn.count("b") / 200 < 0.65                  # one file of "b" is drawn as often as four of "a"
    batch = voc.collate_fn([voc[0], voc[4]])
    assert batch["audio"].shape == (2, 4000) and batch["audio_8000"].shape == (2, 2000) and float(batch["audio"].abs().max()) == pytest.approx(0.475, abs=1e-3)

    tok = CharTokenizer(list("abcdefghijklmnopqrstuvwxyz .0123456789"))
    ds = MagpieTTSDataset(meta, sr, {"en": tok}, codec_frame_rate=25.0, context_duration_min=0.2, context_duration_max=0.4, prior_scaling_factor=0.5)
    b = ds.collate_fn([ds[0], ds[4]])
    assert b["text"].shape[0] == 2 and b["audio"].shape == (2, sr) and 0.2 * sr - 2 <= b["context_audio"].shape[1] <= 0.4 * sr + 2
    assert b["align_prior_matrix"].shape == (2, 25, int(b["text_lens"].max())) and torch.allclose(b["align_prior_matrix"][0].sum(-1), torch.ones(25), atol=1e-4)
    assert len(MagpieTTSDataset.as_model_batch(b)) == 6 and int(b["text"][0, 0]) == tok.vocab_size
    dpo = MagpieTTSDatasetDPO({"a": meta["a"]}, sr, {"en": tok})
    pair = dpo.collate_fn([dpo[0], dpo[1]])
    assert len(dpo) == 2 and pair["rewards"].tolist() == [[1.0, 0.0], [1.0, 0.0]] and pair["chosen"]["audio"].shape == pair["rejected"]["audio"].shape
    long_manifest = tmp_path / "long.json"
    long_manifest.write_text(json.dumps({"text": "one two three. " * 30, "context_audio_filepath": "a0.wav", "language": "en"}))
    inf = ChunkedTTSInferenceDataset({"x": {"manifest_path": str(long_manifest), "audio_dir": str(tmp_path)}}, sr, {"en": tok}, max_chunk_chars=120)
    item = inf.collate_fn([inf[0]])
    assert len(item["chunked_tokens"][0]) >= 3 and all(len(c) <= 123 for c in item["chunked_tokens"][0]) and "context_audio" in item
    assert LanguageThresholds().exceeds_threshold("字" * 101, "zh") and not LanguageThresholds().exceeds_threshold("short text", "en")

    mel = MelSpectrogramFeaturizer(sample_rate=sr, mel_dim=20, win_length=512, hop_length=128)
    entry = {"audio_filepath": "a0.wav"}
    feat_dir = tmp_path / "feats"
    for fz in (mel, EnergyFeaturizer(mel), PitchFeaturizer(sample_rate=sr, win_length=1024, hop_length=128)):
        fz.save(entry, str(tmp_path), str(feat_dir))
    ex = {**mel.load(entry, str(tmp_path), str(feat_dir)), **EnergyFeaturizer(mel).load(entry, str(tmp_path), str(feat_dir)),
          **PitchFeaturizer(sample_rate=sr, win_length=1024, hop_length=128).load(entry, str(tmp_path), str(feat_dir)), "speaker": "a"}
    assert ex["mel_spec"].shape == (20, 126) and ex["energy"].shape == (126,)
    voiced = ex["voiced_mask"][8:-8]
    assert bool(voiced.all()) and float((ex["pitch"][8:-8] - 200.0).abs().max()) < 2.0               # the 200 Hz tone is found
    noise_pitch = PitchFeaturizer(sample_rate=sr, win_length=1024, hop_length=128).compute_pitch(torch.randn(8000) * 0.1)
    assert float(noise_pitch[1].float().mean()) < 0.2                                                 # noise is unvoiced
    stats = tmp_path / "stats.json"
    stats.write_text(json.dumps({"default": {"pitch_mean": 100.0, "pitch_std": 50.0}, "a": {"pitch_mean": 200.0, "pitch_std": 10.0}}))
    e1, e2 = dict(ex), dict(ex)
    MeanVarianceNormalization("pitch", str(stats)).process(e1)
    MeanVarianceSpeakerNormalization("pitch", str(stats)).process(e2)
    assert float(e1["pitch"][20]) == pytest.approx(2.0, abs=0.05) and abs(float(e2["pitch"][20])) < 0.2
    e3 = {"energy": ex["energy"].clone()}
    LogCompression("energy").process(e3)
    assert torch.allclose(e3["energy"], torch.log(ex["energy"] + 1.0))
    assert torch.allclose(mel.collate_fn([{"mel_spec": ex["mel_spec"]}, {"mel_spec": ex["mel_spec"][:, :100]}])["mel_spec"][1, :, 100:], torch.zeros(20, 26))

    sig = np.concatenate([np.zeros(8000), 0.5 * np.sin(2 * np.pi * 200 * t[:8000]), np.zeros(8000)]).astype(np.float32)
    trimmed, s, e = EnergyAudioTrimmer(db_threshold=30.0, pad_seconds=0.05, trim_win_length=512, trim_hop_length=128).trim_audio(sig, sr)
    assert 6500 <= s <= 8000 and 16000 <= e <= 17500 and len(trimmed) == e - s
    vad = lambda frames: (frames.abs().amax(dim=1) > 0.1).float()  # noqa: E731
    _, s2, e2_ = VadAudioTrimmer(vad, vad_sample_rate=8000, trim_win_length=256, trim_hop_length=64, pad_seconds=0.0).trim_audio(sig, sr)
    assert 7000 <= s2 <= 8100 and 15900 <= e2_ <= 17000
    assert float(np.abs(normalize_volume(sig, 0.5)).max()) == pytest.approx(0.5)
    p = BetaBinomialInterpolator()(37, 12)
    assert p.shape == (37, 12) and int(p[0].argmax()) == 0 and int(p[-1].argmax()) == 11


def test_seanet_codec_and_residual_vector_quantisers():
    from speech_b200.tts.encodec_modules import EuclideanCodebook, GroupResidualVectorQuantizer, ResidualVectorQuantizer, SEANetDecoder, SEANetEncoder

    torch.manual_seed(0)
    enc = SEANetEncoder(down_sample_rates=(2, 4), base_channels=4, encoded_dim=8, rnn_layers=1)
    dec = SEANetDecoder(up_sample_rates=(4, 2), base_channels=16, encoded_dim=8, rnn_layers=1)
    audio, alen = torch.randn(2, 160), torch.tensor([160, 120])
    z, zl = enc(audio, alen)
    assert z.shape == (2, 8, 20) and zl.tolist() == [20, 15] and float(z[1, :, 15:].abs().sum()) == 0.0
    y, yl = dec(z, zl)
    assert y.shape == (2, 160) and yl.tolist() == [160, 120] and float(y[1, 120:].abs().sum()) == 0.0
    # padding does not change the valid part
    z2, _ = enc(torch.cat([audio[1:, :120], torch.randn(1, 40)], 1), torch.tensor([120]))
    assert torch.allclose(z2[0, :, :15], z[1, :, :15], atol=1e-5)
    # codebook: k-means start on the first batch, EMA pull towards the data, dead codes re-seeded
    cb = EuclideanCodebook(16, 4, decay=0.8, threshold_ema_dead_code=0.5, kmeans_iters=5).train()
    cents = torch.randn(4, 4) * 5
    x = (cents[torch.randint(0, 4, (2, 50))] + 0.05 * torch.randn(2, 50, 4)).transpose(1, 2)
    lens = torch.tensor([50, 40])
    for _ in range(10):
        deq, idx, commit = cb(x, lens)
    assert bool(cb.initialized) and float(commit) < 0.05 and idx.shape == (2, 50) and int(idx[1, 40:].abs().sum()) == 0
    assert float((cb.decode(cb.encode(x, lens), lens) - x)[0].pow(2).mean()) < 0.05
    xg = x.clone().requires_grad_(True)
    cb(xg, lens)[0].sum().backward()
    assert torch.allclose(xg.grad[0], torch.ones_like(xg.grad[0]))                     # straight-through
    rvq = ResidualVectorQuantizer(num_codebooks=3, codebook_size=16, codebook_dim=4, kmeans_iters=3).train()
    feats = torch.randn(2, 4, 30)
    fl = torch.tensor([30, 20])
    for _ in range(5):
        q, ids = rvq(feats, fl)
    assert ids.shape == (3, 2, 30) and float(rvq.commit_loss) > 0
    rvq.eval()
    ids = rvq.encode(feats, fl)
    errs = [float((sum(b.decode(ids[k], fl) for k, b in enumerate(rvq.books[: n + 1])) - feats)[0].pow(2).mean()) for n in range(3)]
    assert errs[0] > errs[1] > errs[2] and torch.allclose(rvq.decode(ids, fl), rvq(feats, fl)[0].detach(), atol=1e-5)
    g = GroupResidualVectorQuantizer(num_codebooks=4, num_groups=2, codebook_size=16, codebook_dim=8, kmeans_iters=2).train()
    q, ids = g(torch.randn(2, 8, 12), torch.tensor([12, 9]))
    assert q.shape == (2, 8, 12) and ids.shape == (4, 2, 12) and g.decode(ids, torch.tensor([12, 9])).shape == (2, 8, 12)


def test_magpie_helpers_special_tokens_frames_and_char_aware_encoder():
    from speech_b200.tts.magpie_helpers import (CharAwareSubwordEncoder, EOSDetectionMethod, SpecialAudioToken, add_special_tokens, build_vocabs,
                                                clear_forbidden_logits, cosine_schedule, pad_audio_codes, remove_special_tokens)

    N = 100
    assert SpecialAudioToken.get_index(SpecialAudioToken.AUDIO_EOS, N) == 101 and len(SpecialAudioToken.get_forbidden_tokens(N)) == 7
    lg = clear_forbidden_logits(torch.zeros(1, 2, N + 8), N)
    assert torch.isinf(lg[0, 0, 100]) and lg[0, 0, 101] == 0 and torch.isinf(lg[0, 1, 104:]).all()
    assert torch.isinf(clear_forbidden_logits(torch.zeros(1, 1, N + 8), N, forbid_audio_eos=True)[0, 0, 101])
    codes = torch.arange(1, 11).view(1, 2, 5).repeat(2, 1, 1)
    lens = torch.tensor([5, 3])
    with_tok, l2 = add_special_tokens(codes, lens, bos_id=100, eos_id=101)
    assert l2.tolist() == [7, 5] and with_tok[0, 0].tolist() == [100, 1, 2, 3, 4, 5, 101] and with_tok[1, 1, :5].tolist() == [100, 6, 7, 8, 101]
    back, l3 = remove_special_tokens(with_tok, l2)
    assert l3.tolist() == [5, 3] and torch.equal(back[0], codes[0]) and back[1, 0, :3].tolist() == [1, 2, 3] and int(back[1, :, 3:].sum()) == 0
    assert pad_audio_codes(codes, 4).shape == (2, 2, 8) and pad_audio_codes(codes, 5) is codes
    assert float(cosine_schedule(torch.tensor(0.0))) == 1.0 and float(cosine_schedule(torch.tensor(1.0))) < 1e-6
    am, sm = torch.tensor([[5, 101], [5, 5]]), torch.tensor([[5, 5], [101, 5]])
    assert EOSDetectionMethod.ARGMAX_ANY.detect(am, sm, 101).tolist() == [True, False]
    assert EOSDetectionMethod.ARGMAX_OR_MULTINOMIAL_ANY.detect(am, sm, 101).tolist() == [True, True]
    assert EOSDetectionMethod.ARGMAX_OR_MULTINOMIAL_ZERO_CB.detect(am, sm, 101).tolist() == [False, True]
    assert EOSDetectionMethod.ARGMAX_ALL.detect(am, sm, 101).tolist() == [False, False]
    vocab = {"<pad>": 0, "▁the": 1, "▁then": 2, "ing": 3, "<bos>": 4, "▁zebra": 5}
    table, chars = build_vocabs(vocab, 0)
    assert table[1] == [chars[" "], chars["t"], chars["h"], chars["e"]] and table[4] == [chars["<bos>"]] and 0 not in table
    torch.manual_seed(0)
    enc = CharAwareSubwordEncoder(16, vocab, 0, n_layers=1, n_heads=2).eval()
    ids = torch.tensor([[1, 2, 5, 0], [3, 1, 0, 0]])
    e = enc(ids, ids != 0)
    assert e.shape == (2, 4, 16) and float(e[0, 3].abs().sum()) == 0.0 and torch.allclose(e[0, 0], e[1, 1])
    cos = torch.nn.functional.cosine_similarity
    assert float(cos(e[0, 0], e[0, 1], dim=0)) > float(cos(e[0, 0], e[0, 2], dim=0))       # "the" is closer to "then" than to "zebra"


def test_tts_logging_callback_writes_audio_and_images(tmp_path):
    from speech_b200.tts.callbacks import AudioCodecArtifactGenerator, LoggingCallback, VocoderArtifactGenerator, create_id, write_pgm
    from speech_b200.tts.classic import HifiGanModel

    torch.manual_seed(0)
    codec = AudioCodecModel(OmegaConf.create(CODEC_CFG))
    audio, lens = torch.randn(2, 2048) * 0.1, torch.tensor([2048, 1536])
    loader = [{"audio": audio, "audio_lens": lens, "audio_filepaths": ["spk1/a.wav", "spk2/b.wav"]}]

    class FakeTrainer:
        current_epoch, global_step, is_global_zero = 0, 10, True

    class FakeBoard:
        def __init__(self):
            self.audio, self.images = [], []

        def add_audio(self, tag, data, global_step, sample_rate):
            self.audio.append((tag, global_step, sample_rate))

        def add_image(self, tag, data, global_step):
            self.images.append((tag, data.shape))

    board = FakeBoard()
    cb = LoggingCallback([AudioCodecArtifactGenerator(log_audio=True, log_encoding=True, log_dequantized=True)], loader, epoch_frequency=2,
                         output_dir=str(tmp_path / "logs"), loggers=[board])
    tr = FakeTrainer()
    cb.on_train_epoch_end(tr, codec)
    d = tmp_path / "logs" / "epoch_0"
    names = sorted(os.listdir(d))
    assert names == ["deq_spk1_a.pgm", "deq_spk2_b.pgm", "enc_spk1_a.pgm", "enc_spk2_b.pgm", "gt_spk1_a.wav", "gt_spk2_b.wav", "pred_spk1_a.wav", "pred_spk2_b.wav"]
    assert open(d / "enc_spk1_a.pgm", "rb").read(2) == b"P5" and len(board.audio) == 4 and board.images[0][1][0] == 1 and codec.training
    tr.current_epoch = 1
    cb.on_train_epoch_end(tr, codec)                                   # off-frequency epoch: nothing
    assert not (tmp_path / "logs" / "epoch_1").exists()
    tr.current_epoch = 2
    cb.on_train_epoch_end(tr, codec)                                   # later logs skip the ground truth
    assert sorted(os.listdir(tmp_path / "logs" / "epoch_2")) == ["deq_spk1_a.pgm", "deq_spk2_b.pgm", "enc_spk1_a.pgm", "enc_spk2_b.pgm", "pred_spk1_a.wav", "pred_spk2_b.wav"]
    voc = HifiGanModel(OmegaConf.create({"sample_rate": 8000, "generator": {"input_dim": 20, "up_sample_rates": [4, 4, 4], "base_channels": 16, "resblock_kernel_sizes": [3]},
                                         "discriminator": {"periods": [2], "stft_resolutions": [[256, 64, 256]]}, "mel": {"n_fft": 256, "hop": 64, "win": 256}}))
    cb2 = LoggingCallback([VocoderArtifactGenerator()], [(audio, lens)], log_epochs=[5], output_dir=str(tmp_path / "voc"))
    tr.current_epoch = 5
    cb2.on_train_epoch_end(tr, voc)
    assert sorted(os.listdir(tmp_path / "voc" / "epoch_5")) == ["gt_item0.wav", "gt_item1.wav", "voc_item0.wav", "voc_item1.wav"]
    assert create_id("/data/x/y.wav") == "data_x_y"
    write_pgm(str(tmp_path / "flat.pgm"), np.zeros((3, 4)))
    assert len(open(tmp_path / "flat.pgm", "rb").read()) == len(b"P5\n4 3\n255\n") + 12


def test_tts_text_tokenizers():
    from speech_b200.tokenizers.tts import (AggregatedTTSTokenizer, ArabicCharsTokenizer, EnglishCharsTokenizer, EnglishPhonemesTokenizer, FrenchCharsTokenizer,
                                            GermanCharsTokenizer, HindiCharsTokenizer, IPATokenizer, SpanishCharsTokenizer, english_text_preprocessing,
                                            get_grapheme_character_set, get_ipa_punctuation_list)
    from speech_b200.tts.g2p import IpaG2p

    assert english_text_preprocessing("Café “naïve”… ok") == 'cafe "naive"... ok'
    assert "Ñ" in get_grapheme_character_set("es-ES") and "ñ" in get_grapheme_character_set("es-ES", "mixed") and "¿" in get_ipa_punctuation_list("es-ES")
    with pytest.raises(ValueError):
        get_grapheme_character_set("xx-XX")
    en = EnglishCharsTokenizer(pad_with_space=True, add_blank_at="last_but_one")
    ids = en("Hello,   Wörld§!")
    assert en.decode(ids) == " hello, world! " and en.pad == len(en.tokens) - 3 and en.blank == en.pad + 1 and en.oov == en.pad + 2
    last = EnglishCharsTokenizer(add_blank_at="last")
    assert last.blank == len(last.tokens) - 1 and last.oov == len(last.tokens) - 2
    nop = EnglishCharsTokenizer(punct=False)
    assert nop.decode(nop("hi, there!")) == "hi there"
    assert GermanCharsTokenizer().decode(GermanCharsTokenizer()("Straße und Öl")) == "Straße und Öl"
    assert SpanishCharsTokenizer().decode(SpanishCharsTokenizer()("¿Qué Niño?")) == "¿qué niño?"
    assert FrenchCharsTokenizer().decode(FrenchCharsTokenizer()("Ça va, garçon")) == "ça va, garçon"
    assert HindiCharsTokenizer().decode(HindiCharsTokenizer()("नमस्ते।")) == "नमस्ते।" and len(ArabicCharsTokenizer()("مرحبا؟")) == 6
    arpa = {"hello": ["HH", "AH0", "L", "OW1"], "world": ["W", "ER1", "L", "D"]}

    def g2p(text):
        out = []
        for tok in re.findall(r"\w+|[^\w\s]|\s+", text):
            out += [" "] if tok.isspace() else arpa.get(tok.lower(), list(tok.lower()) if tok.isalpha() else [tok])
        return out

    ph = EnglishPhonemesTokenizer(g2p, stresses=True, chars=True)
    ids = ph("Hello xyz, world")
    assert ph.decode(ids) == "HH|AH0|L|OW1| |x|y|z|,| |W|ER1|L|D"
    ns = EnglishPhonemesTokenizer(g2p, stresses=False)
    assert ns.decode(ns("hello world")) == "HH|AH|L|OW| |W|ER|L|D" and ns.vocab_size < ph.vocab_size
    ipa_g2p = IpaG2p({"hello": ["həˈloʊ"], "world": ["ˈwɝld"]}, use_chars=True, grapheme_prefix="#")
    ipa = IPATokenizer(ipa_g2p, locale="en-US")
    assert ipa.decode(ipa("hello xy world!")) == "həˈloʊ #X#Y ˈwɝld!" and "#Q" in ipa.tokens
    fixed = IPATokenizer(IpaG2p({"hello": ["həˈloʊ"], "yes": ["jɛs"]}, use_chars=True, grapheme_prefix="#"), locale=None, fixed_vocab=list("həˈloʊ") + ["#Y", "#E", "#S"])
    assert fixed.decode(fixed("hello yes")) == "həˈloʊ #Y#E#S"                  # "jɛs" uses symbols outside the fixed inventory: spelled instead
    agg = AggregatedTTSTokenizer([en, ipa], ["english_chars", "english_ipa"])
    a, b = agg.encode("hello", "english_chars"), agg.encode("hello", "english_ipa")
    assert max(a) < en.vocab_size <= min(b) and agg.vocab_size == en.vocab_size + ipa.vocab_size and agg.decode(b, "english_ipa") == "həˈloʊ"


def test_hybrid_decoder_moe_block_routes_by_group_and_matches_dense_evaluation():
    """The mixture-of-experts block of the hybrid decoder: group-limited sigmoid routing, the sorted-by-expert evaluation equal to a
    per-token dense evaluation, incremental decoding equal to the full pass."""
    import torch
    import torch.nn.functional as F

    from speech_b200.speechlm.llm import LLMConfig
    from speech_b200.tts.easy_magpie import NemotronHDecoder, NemotronHMoE

    torch.manual_seed(0)
    moe = NemotronHMoE(16, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=12, moe_shared_expert_intermediate_size=20, n_group=4,
                       topk_group=1, routed_scaling_factor=1.5, initializer_range=0.5, mlp_hidden_act="relu2")
    x = torch.randn(3, 5, 16)
    idx, w = moe.route(x.reshape(-1, 16))
    assert idx.shape == (15, 2) and bool((idx[:, 0] // 2 == idx[:, 1] // 2).all())      # one eligible group of two experts → both from it
    assert torch.allclose(w.sum(-1), torch.full((15,), 1.5), atol=1e-5)
    scores = F.linear(x.reshape(-1, 16), moe.router).sigmoid()
    best_group = scores.view(15, 4, 2).sum(-1).argmax(-1)
    assert torch.equal(best_group, idx[:, 0] // 2)
    y = moe(x)
    ref = torch.zeros(15, 16)
    h = x.reshape(-1, 16)
    for n in range(15):
        for j in range(2):
            e = int(idx[n, j])
            ref[n] += w[n, j] * F.linear(F.relu(F.linear(h[n], moe.up[e])).square(), moe.down[e])
    ref = ref + moe.shared_down(F.relu(moe.shared_up(h)).square())
    assert torch.allclose(y.reshape(15, 16), ref, atol=1e-4)
    moe.e_score_correction_bias[5] = 10.0                          # the load-balancing bias steers the choice, not the weight
    idx2, w2 = moe.route(h)
    assert bool((idx2 == 5).any(-1).all()) and torch.allclose(w2.sum(-1), torch.full((15,), 1.5), atol=1e-5)
    y.sum().backward()
    assert moe.router.grad is not None and moe.up.grad.abs().sum() > 0

    tiny = dict(vocab_size=32, hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1)
    dec = NemotronHDecoder(LLMConfig(**tiny), "ME*", {"d_state": 8, "head_dim": 8}, {"n_routed_experts": 4, "moe_intermediate_size": 8,
                                                                                  "moe_shared_expert_intermediate_size": 8}, num_layers=5).eval()
    assert dec.pattern == "ME*ME"
    z = torch.randn(2, 6, 16)
    with torch.no_grad():
        full = dec(z)
        cache = dec.new_cache()
        steps = torch.cat([dec(z[:, t:t + 1], cache) for t in range(6)], dim=1)
    assert torch.allclose(full, steps, atol=1e-4)


def test_tts_submodules_masking_conditioning_and_speaker_encoder():
    import torch

    from speech_b200.tts import submodules as S

    torch.manual_seed(0)
    x = torch.randn(2, 4, 10)
    mask = (torch.arange(10)[None, :] < torch.tensor([10, 6])[:, None]).unsqueeze(1).float()
    norm = S.MaskedInstanceNorm1d(4)
    y = norm(x, mask)
    assert torch.allclose(y[1, :, :6].mean(-1), torch.zeros(4), atol=1e-5) and torch.allclose(y[1, :, :6].std(-1), torch.ones(4), atol=1e-4) and float(y[1, :, 6:].abs().sum()) == 0
    y2 = norm(torch.cat([x[1:, :, :6], torch.full((1, 4, 4), 50.0)], dim=-1), mask[1:])       # padding values do not matter
    assert torch.allclose(y2[0, :, :6], y[1, :, :6], atol=1e-5)

    pc = S.PartialConv1d(4, 3, 3, padding=1)
    full = pc(x[1:, :, :6], torch.ones(1, 1, 6))
    part = pc(x[1:], mask[1:])
    plain = torch.nn.functional.conv1d(x[1:, :, :6], pc.weight, pc.bias, padding=1)
    assert torch.allclose(full[..., 1:5], plain[..., 1:5], atol=1e-5)                      # interior windows are an ordinary convolution
    assert torch.allclose(part[..., :6], full, atol=1e-5) and float(part[..., 7:].abs().sum()) == 0
    edge = (plain[..., 0] - pc.bias) * 1.5 + pc.bias                                        # 2 of 3 taps valid → scaled by 3/2
    assert torch.allclose(full[..., 0], edge, atol=1e-5)

    cn = S.ConvNorm(4, 5, 3, use_partial_padding=True, norm_fn=S.MaskedInstanceNorm1d)
    assert cn(x, mask).shape == (2, 5, 10) and float(cn(x, mask)[1, :, 6:].abs().sum()) == 0
    with pytest.raises(ValueError):
        S.ConvNorm(4, 5, 4)

    pre = S.Prenet(6, [8, 8], p_dropout=0.5).eval()
    a, b = pre(torch.ones(3, 6)), pre(torch.ones(3, 6))
    assert not torch.equal(a, b)                                                             # dropout stays on in eval mode
    c = pre(torch.ones(3, 6), inference=True)
    assert torch.equal(c[0], c[1])                                                            # one mask for the batch

    att = S.Attention(7, 5, 6, 4, 3)
    mem = torch.randn(2, 9, 5)
    pad = torch.arange(9)[None, :] >= torch.tensor([9, 4])[:, None]
    ctx, w = att(torch.randn(2, 7), mem, att.memory_layer(mem), torch.rand(2, 2, 9), pad)
    assert ctx.shape == (2, 5) and torch.allclose(w.sum(1), torch.ones(2), atol=1e-5) and float(w[1, 4:].sum()) == 0

    cond = torch.randn(2, 1, 3)
    h = torch.randn(2, 5, 8)
    cln = S.ConditionalLayerNorm(8, 3, ["layernorm"])
    assert torch.allclose(cln(h, cond), torch.nn.functional.layer_norm(h, (8,)), atol=1e-6)  # identity at initialisation
    with pytest.raises(ValueError):
        cln(h)
    assert torch.equal(S.ConditionalInput(8, 3, [])(h), h)
    ci = S.ConditionalInput(8, 3, ["add", "concat"])
    assert ci(h, cond).shape == h.shape
    with pytest.raises(ValueError):
        S.ConditionalInput(8, 3, ["multiply"])

    ref = S.ReferenceEncoder(n_mels=16, cnn_filters=[4, 8], dropout=0.0, gru_hidden=12)
    mel = torch.randn(2, 16, 20)
    lens = torch.tensor([20, 11])
    r = ref(mel, lens)
    r_short = ref(mel[1:, :, :11], lens[1:])
    assert r.shape == (2, 12) and torch.allclose(r[1], r_short[0], atol=1e-5)               # padding does not change the summary
    gst = S.GlobalStyleToken(ref, gst_size=12, n_style_token=5, n_style_attn_head=3)
    assert gst(mel, lens).shape == (2, 12)
    enc = S.SpeakerEncoder(S.SpeakerLookupTable(4, 12), gst)
    both = enc(speaker=torch.tensor([1, 3]), reference_spec=mel, reference_spec_lens=lens)
    only = enc(speaker=torch.tensor([1, 3]))
    assert both.shape == (2, 1, 12) and torch.allclose(both - only, gst(mel, lens).unsqueeze(1), atol=1e-5) and enc() is None
    enc.overwrite_precomputed_emb(torch.arange(12.0))
    assert torch.equal(enc(batch_size=3)[2, 0], torch.arange(12.0))


def test_fastpitch_with_speaker_encoder_conditions_on_reference():
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.tts.classic import FastPitchModel

    torch.manual_seed(0)
    cfg = OmegaConf.create({"n_symbols": 20, "symbols_embedding_dim": 16, "n_mel_channels": 16, "d_inner": 32, "encoder_layers": 1, "decoder_layers": 1, "sample_rate": 8000,
                            "n_fft": 128, "hop_length": 32, "win_length": 128,
                            "speaker_encoder": {"lookup_module": {"n_speakers": 3}, "gst_module": {"n_mels": 16, "cnn_filters": [4, 4], "n_style_token": 4, "n_style_attn_head": 2}}})
    m = FastPitchModel(cfg).eval()
    toks = torch.randint(1, 20, (1, 7))
    lens = torch.tensor([7])
    ref_a, ref_b = torch.randn(1, 16, 30), torch.randn(1, 16, 30)
    with torch.no_grad():
        e0 = m.speaker_encoder(batch_size=1, speaker=torch.tensor([0]), reference_spec=ref_a, reference_spec_lens=torch.tensor([30]))
        e1 = m.speaker_encoder(batch_size=1, speaker=torch.tensor([2]), reference_spec=ref_b, reference_spec_lens=torch.tensor([30]))
        out = m(toks, lens, speaker=torch.tensor([0]), reference_spec=ref_a, reference_spec_lens=torch.tensor([30]))
    assert e0.shape == (1, 1, 16) and not torch.allclose(e0, e1) and out["mel"].shape[1] == 16


def test_codec_spectral_encoders_resnet_decoder_and_codec_model_with_them():
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.tts import audio_codec_encoders as E
    from speech_b200.tts.audio_codec import AudioCodecModel

    torch.manual_seed(0)
    audio = torch.randn(2, 4096) * 0.1
    lens = torch.tensor([4096, 3000])
    audio[1, 3000:] = 0

    act = E.CodecActivation("half_snake", 6)
    z = torch.randn(1, 6, 5)
    assert torch.allclose(act(z)[:, :3], z[:, :3] + torch.sin(z[:, :3]).square(), atol=1e-5) and torch.allclose(act(z)[:, 3:], torch.nn.functional.leaky_relu(z[:, 3:], 0.01))
    pre = E.PreEmphasis(0.5)(torch.tensor([[1.0, 2.0, 4.0]]))
    assert pre.tolist() == [[0.0, 1.5, 3.0]]

    stft = E.STFTProcessor(256, 256, 64)
    s, sl = stft(audio, lens)
    assert s.shape == (2, 129, 64) and sl.tolist() == [64, 46] and float(s[1, :, 46:].abs().sum()) == 0
    melp = E.MelSpectrogramProcessor(16000, 256, 64, mel_dim=20)
    m, ml = melp(audio, lens)
    assert m.shape == (2, 20, 64) and ml.tolist() == [64, 46] and bool((m[0] >= 0).all())     # log(1 + mel) ≥ 0

    with pytest.raises(ValueError):
        E.MultiBandMelEncoder([(0, 8), (10, 20)], melp, out_channels=4)
    mb = E.MultiBandMelEncoder([(0, 8), (8, 20)], melp, out_channels=4, num_layers=1, hidden_channels=8, filters=16)
    enc, el = mb(audio, lens)
    assert enc.shape == (2, 8, 64) and el.tolist() == [64, 46] and mb.total_stride == 64 and float(enc[1, :, 46:].abs().sum()) == 0
    fb = E.FullBandMelEncoder(melp, E.ResNetEncoder(20, 6, num_layers=1, hidden_channels=8, filters=16))
    assert fb(audio, lens)[0].shape == (2, 6, 64)

    with pytest.raises(ValueError):
        E.MultiResolutionSTFTEncoder(8, [(128, 32, 128), (256, 96, 256)], [8, 8])
    mr = E.MultiResolutionSTFTEncoder(8, [(128, 32, 128), (256, 64, 256), (512, 128, 512)], [8, 12, 16], down_sample_filter_list=[16], down_sample_rate_list=[2])
    enc, el = mr(audio, lens)
    assert mr.total_stride == 256 and enc.shape == (2, 8, 16) and el.tolist() == [16, 11]

    ce = E.CausalHiFiGANEncoder(6, down_sample_rates=(2, 4), base_channels=4, resblock_kernel_sizes=(3,), resblock_dilation_sizes=(1, 2))
    a, al = ce(audio[:1, :512], torch.tensor([512]))
    a2, _ = ce(torch.cat([audio[:1, :256], torch.randn(1, 256)], dim=1), torch.tensor([512]))
    assert a.shape == (1, 6, 64) and torch.allclose(a[..., :32], a2[..., :32], atol=1e-5)        # no look-ahead

    dec = E.ResNetDecoder(8, 12, [2], [10], 2, 16, [4, 2], [8, 4], resblock_up_sample_kernel_size=5)
    y, yl = dec(torch.randn(2, 8, 10), torch.tensor([10, 7]))
    assert dec.total_stride == 16 and y.shape == (2, 160) and yl.tolist() == [160, 112] and float(y[1, 112:].abs().sum()) == 0 and float(y.abs().max()) <= 1
    cdec = E.ResNetDecoder(8, 12, [2], [10], 1, 16, [4], [6], is_causal=True).eval()
    x = torch.randn(1, 8, 12)
    x2 = torch.cat([x[..., :6], torch.randn(1, 8, 6)], dim=-1)
    with torch.no_grad():
        y1, _ = cdec(x, torch.tensor([12]))
        y2, _ = cdec(x2, torch.tensor([12]))
    assert torch.allclose(y1[:, :48], y2[:, :48], atol=1e-5) and not torch.allclose(y1[:, 48:], y2[:, 48:])
    mr.post_conv.remove_weight_norm()
    assert not torch.nn.utils.parametrize.is_parametrized(mr.post_conv.conv)

    mpd = E.MultiPeriodDiscriminator((2, 3))
    sr, sg, fr, fg = mpd(audio[:, :600], audio[:, :600] * 0.5)
    assert len(sr) == len(sg) == 2 and len(fr[0]) == len(fg[0])

    cfg = OmegaConf.create({"sample_rate": 16000, "train_discriminator": False, "mel_loss": {"n_mels": 16, "n_fft": 256, "hop": 64, "win": 256},
                            "audio_encoder": {"_target_": "speech_b200.tts.audio_codec_encoders.MultiBandMelEncoder", "mel_bands": [[0, 8], [8, 16]], "out_channels": 4,
                                              "num_layers": 1, "hidden_channels": 8, "filters": 8,
                                              "mel_processor": {"sample_rate": 16000, "win_length": 256, "hop_length": 64, "mel_dim": 16}},
                            "vector_quantizer": {"num_groups": 2, "num_levels_per_group": [4, 4, 4, 4]},
                            "audio_decoder": {"_target_": "speech_b200.tts.audio_codec_encoders.ResNetDecoder", "input_dim": 8, "input_filters": 8, "pre_up_sample_rates": [2],
                                              "pre_up_sample_filters": [8], "n_hidden_layers": 1, "hidden_filters": 8, "resblock_up_sample_rates": [8, 4],
                                              "resblock_up_sample_filters": [6, 4]}})
    model = AudioCodecModel(cfg).eval()
    assert model.samples_per_frame == 64
    with torch.no_grad():
        toks, tl = model.encode(audio, lens)
        rec, rl = model.decode(toks, tl)
    assert toks.shape == (2, 2, 64) and tl.tolist() == [64, 46] and rec.shape == (2, 4096) and rl.tolist() == [4096, 2944]


def test_tts_base_kinds_text_normaliser_hook_and_griffin_lim_vocoder():
    import math

    import numpy as np
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.modules.preprocessor import mel_filterbank
    from speech_b200.tts.base import GriffinLimVocoder, SpectrogramGenerator, Vocoder
    from speech_b200.tts.classic import FastPitchModel, HifiGanModel

    assert issubclass(FastPitchModel, SpectrogramGenerator) and issubclass(HifiGanModel, Vocoder)
    with pytest.raises(TypeError):
        SpectrogramGenerator(OmegaConf.create({}))                                          # abstract: parse / generate_spectrogram missing
    cfg = OmegaConf.create({"n_symbols": 40, "symbols_embedding_dim": 16, "n_mel_channels": 16, "d_inner": 32, "encoder_layers": 1, "decoder_layers": 1,
                            "sample_rate": 8000, "n_fft": 128, "hop_length": 32, "win_length": 128})
    m = FastPitchModel(cfg, tokenizer=type("Tok", (), {"text_to_ids": staticmethod(lambda t: [1 + (ord(c) % 30) for c in t])})())
    raw = m.parse("ab 12")
    m.text_normalizer_call = lambda t, verbose=False: t.replace("12", "twelve")
    m.text_normalizer_call_kwargs = {"verbose": False}
    assert m.parse("ab 12").shape[1] == raw.shape[1] + 4 and m.parse("ab 12", normalize=False).shape == raw.shape

    sr, n_fft, hop = 8000, 512, 128
    t = torch.arange(sr) / sr
    x = 0.5 * torch.sin(2 * math.pi * 440 * t)
    win = torch.hann_window(n_fft)
    mag = torch.stft(x, n_fft, hop, n_fft, win, return_complex=True).abs()
    fb = torch.as_tensor(np.asarray(mel_filterbank(sr, n_fft, 64, 0.0, None)), dtype=torch.float32)
    logmel = torch.log(torch.matmul(fb, mag).clamp(min=1e-5))[None]
    voc = GriffinLimVocoder(sr, n_fft, hop, n_mels=64, n_iters=16)
    y = voc.convert_spectrogram_to_audio(logmel)
    assert y.shape[0] == 1 and abs(y.shape[1] - sr) <= hop
    spec_y = torch.stft(y[0], n_fft, hop, n_fft, win, return_complex=True).abs().mean(-1)
    assert abs(int(spec_y.argmax()) - round(440 / (sr / n_fft))) <= 1                      # the tone survives the mel → waveform inversion
    assert float(y[0, 1000:-1000].pow(2).mean().sqrt()) == pytest.approx(0.5 / math.sqrt(2), rel=0.3)


def test_heteronym_disambiguation_picks_the_pronunciation_the_audio_supports():
    import torch

    from speech_b200.tts.heteronym_aligner import alignment_score, disambiguate_heteronyms

    symbols = [" ", "r", "iy", "eh", "d", "ay", "b", "uh", "k"]
    sid = {s: k for k, s in enumerate(symbols)}

    def aligner(spec, spec_len, text, text_len):
        """Frames are (noisy) one-hot symbol indicators: the log-probability of token u at frame t is the log-softmax over tokens of their match."""
        sim = spec[0].t()[:, text[0]] * 8.0                                  # [T, U]
        logp = torch.log_softmax(sim, dim=-1)[None, None]
        return logp.exp(), logp

    def render(seq, per=4):
        frames = torch.zeros(len(symbols), len(seq) * per)
        for k, s in enumerate(seq):
            frames[sid[s], k * per:(k + 1) * per] = 1.0
        return frames[None] + 0.05 * torch.randn(1, len(symbols), len(seq) * per, generator=torch.Generator().manual_seed(0))

    encode = lambda syms: [sid[s] for s in syms]  # noqa: E731
    prons = {"read": [["r", "iy", "d"], ["r", "eh", "d"]], "i": [["ay"]], "book": [["b", "uh", "k"]]}
    words = ["i", "read", "book"]
    for truth, want in ((["ay", " ", "r", "eh", "d", " ", "b", "uh", "k"], 1), (["ay", " ", "r", "iy", "d", " ", "b", "uh", "k"], 0)):
        spec = render(truth)
        slen = torch.tensor([spec.shape[-1]])
        chosen, dec = disambiguate_heteronyms(aligner, spec, slen, words, prons, encode)
        assert len(dec) == 1 and dec[0]["word"] == "read" and dec[0]["choice"] == want and dec[0]["confidence"] > 0
        assert chosen[1] == prons["read"][want] and chosen[0] == ["ay"]
        good, bad = alignment_score(aligner, spec, slen, encode(truth)), alignment_score(aligner, spec, slen, encode(truth[:3] + ["k"] + truth[4:]))
        assert good > bad
    unsure, dec = disambiguate_heteronyms(aligner, spec, slen, words, prons, encode, min_confidence=1e9)
    assert dec[0]["choice"] is None and unsure[1] == prons["read"][0]


def test_fastpitch_adapters_train_alone_and_round_trip(tmp_path):
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.tts.classic import FastPitchModel

    torch.manual_seed(0)
    cfg = OmegaConf.create({"n_symbols": 20, "symbols_embedding_dim": 16, "n_mel_channels": 16, "d_inner": 32, "encoder_layers": 2, "decoder_layers": 1, "sample_rate": 8000,
                            "n_fft": 128, "hop_length": 32, "win_length": 128})
    m = FastPitchModel(cfg).eval()
    toks, lens = torch.randint(1, 20, (2, 7)), torch.tensor([7, 5])
    with torch.no_grad():
        base = m(toks, lens)["mel"]
    acfg = {"in_features": 16, "dim": 8, "activation": "swish", "norm_position": "pre"}
    m.add_adapter("encoder:spk", acfg)
    m.add_adapter("decoder:spk", acfg)
    assert m.get_enabled_adapters() == ["encoder:spk", "decoder:spk"] and len(m.encoder.layers[1].adapter_layer) == 1
    with torch.no_grad():
        fresh = m(toks, lens)["mel"]
    assert torch.allclose(fresh, base, atol=1e-5)                                 # a new adapter starts as the identity
    n = m.freeze_base_and_train_adapters()
    trainable = [k for k, p in m.named_parameters() if p.requires_grad]
    assert n > 0 and all(".adapter_layer." in k for k in trainable) and not m.embedding.weight.requires_grad
    with torch.no_grad():
        for k, p in m.named_parameters():
            if ".adapter_layer." in k:
                p.add_(0.05 * torch.randn_like(p))
        changed = m.eval()(toks, lens)["mel"]
    assert not torch.allclose(changed, base, atol=1e-4)
    m.set_enabled_adapters(enabled=False)
    with torch.no_grad():
        assert torch.allclose(m(toks, lens)["mel"], base, atol=1e-5)              # disabled adapters leave the base model intact
    m.set_enabled_adapters(enabled=True)
    m.save_adapters(str(tmp_path / "spk.pt"))
    torch.manual_seed(0)
    m2 = FastPitchModel(cfg).eval()
    m2.load_state_dict({k: v for k, v in m.state_dict().items() if ".adapter_layer." not in k})
    m2.load_adapters(str(tmp_path / "spk.pt"))
    with torch.no_grad():
        assert torch.allclose(m2(toks, lens)["mel"], changed, atol=1e-5)
    m3 = FastPitchModel(m2.cfg).eval()                                             # the config remembers the adapters: a rebuilt model has them
    assert m3.get_enabled_adapters() == ["encoder:spk", "decoder:spk"]
    with pytest.raises(ValueError):
        m.add_adapter("aligner:spk", acfg)


def test_fastpitch_ssl_trains_on_features_and_swaps_speakers():
    import torch

    from speech_b200.core.config import OmegaConf
    from speech_b200.core.trainer import Trainer
    from speech_b200.tts.base import GriffinLimVocoder
    from speech_b200.tts.fastpitch_ssl import FastPitchModel_SSL

    torch.manual_seed(0)
    cfg = OmegaConf.create({"n_mel_channels": 16, "content_emb_indim": 12, "speaker_emb_indim": 10, "symbols_embedding_dim": 16, "d_inner": 32, "encoder_layers": 1,
                            "decoder_layers": 1, "dropout": 0.0, "train_ds": {"synthetic": {"num_samples": 8}, "batch_size": 4},
                            "validation_ds": {"synthetic": {"num_samples": 4}, "batch_size": 4}, "optim": {"name": "adamw", "lr": 1e-2}})
    voc = GriffinLimVocoder(8000, 128, 32, n_mels=16, n_iters=2, log_input=False)
    model = FastPitchModel_SSL(cfg, vocoder=voc)
    batch = next(iter(model._train_dl))
    first = float(model._losses(batch)[0])
    Trainer(max_steps=12, accelerator="cpu", logger=False, enable_checkpointing=False, log_every_n_steps=100).fit(model)
    model.eval()
    assert float(model._losses(batch)[0]) < first
    ce, cl, spk, mel, ml, dur, pitch = batch
    out, out_len = model.synthesize_spectrogram(ce, spk, cl, durations=dur, pitch=pitch)
    assert out.shape[:2] == (4, 16) and out_len.tolist() == dur.sum(1).long().tolist()                # given durations fix the output length
    other, _ = model.synthesize_spectrogram(ce, spk.flip(0), cl, durations=dur, pitch=pitch)
    assert not torch.allclose(out, other, atol=1e-4)                                                   # another speaker embedding → another voice
    slow, slow_len = model.synthesize_spectrogram(ce, spk, cl, durations=dur, pitch=pitch, pace=0.5)
    assert slow_len.tolist() == (2 * dur.sum(1)).long().tolist()
    free, free_len = model.synthesize_spectrogram(ce, spk, cl)                                         # predicted durations and pitch
    assert free.shape[0] == 4 and int(free_len.min()) >= 0
    wavs = model.generate_wav(ce, spk, cl, durations=dur, pitch=pitch)
    assert len(wavs) == 4 and wavs[0].shape[0] == int(out_len[0]) * (wavs[0].shape[0] // int(out_len[0]))
    assert "vocoder" not in dict(model.named_modules())
