"""Speech-LLM stack on CPU: native decoder-only LM (KV-cache decoding equals full recomputation, HF-directory round trip),
placeholder splicing, LoRA, SALM training + generation, failure detection on the host."""
import math
import os

import pytest
import torch

from speech_b200.core.config import OmegaConf
from speech_b200.core.trainer import Trainer
from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
from speech_b200.parallel.resiliency import FaultToleranceCallback, HeartbeatMonitor, StragglerDetectionCallback
from speech_b200.speechlm.llm import CausalLM, LLMConfig
from speech_b200.speechlm.lora import apply_lora, freeze_and_subset, merge_lora
from speech_b200.speechlm.salm import IGNORE_INDEX, SALM, replace_placeholders_and_build_targets
from speech_b200.tokenizers import ByteLevelTokenizer

TINY = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16)


def test_llm_cache_decode_matches_full_forward_and_left_padding(tmp_path):
    torch.manual_seed(0)
    m = CausalLM(LLMConfig(**TINY)).eval()
    ids = torch.randint(0, 300, (2, 9))
    full = m(input_ids=ids)["logits"]
    cache = [dict() for _ in m.model.layers]
    a = m(input_ids=ids[:, :5], cache=cache)["logits"]
    outs = [a]
    for t in range(5, 9):
        outs.append(m(input_ids=ids[:, t:t + 1], cache=cache)["logits"])
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4)
    # left padding must not change the logits of the real tokens
    pad = torch.cat([torch.zeros(2, 3, dtype=torch.long), ids], dim=1)
    mask = torch.cat([torch.zeros(2, 3, dtype=torch.long), torch.ones(2, 9, dtype=torch.long)], dim=1)
    padded = m(input_ids=pad, attention_mask=mask)["logits"][:, 3:]
    assert torch.allclose(padded, full, atol=1e-4)
    m.save_pretrained(str(tmp_path / "hf"))
    again = CausalLM.from_pretrained(str(tmp_path / "hf")).eval()
    assert torch.allclose(again(input_ids=ids)["logits"], full, atol=1e-6)
    gen = m.generate(input_ids=ids, max_new_tokens=4)
    assert gen.shape == (2, 4)
    ref_next = full[:, -1].argmax(-1)
    assert torch.equal(gen[:, 0], ref_next)


def test_placeholder_splicing_targets_and_left_padding():
    H = 4
    ids = torch.tensor([[5, 99, 6, 7, 0], [99, 8, 99, 0, 0]])          # 99 = audio placeholder, 0 = padding
    emb = torch.arange(2 * 5 * H, dtype=torch.float32).view(2, 5, H)
    tgt = torch.where(ids == 0, torch.full_like(ids, IGNORE_INDEX), ids)
    aud = [torch.full((3, H), -1.0), torch.full((2, H), -2.0), torch.full((1, H), -3.0)]
    e, t, m = replace_placeholders_and_build_targets(ids, emb, 0, 99, aud, tgt)
    assert e.shape == (2, 6, H) and m.sum(1).tolist() == [6, 4]
    assert t[0].tolist() == [5, -100, -100, -100, 6, 7]
    assert t[1].tolist() == [-100, -100, -100, -100, 8, -100]            # left padded: 2 pads, 2 audio, token, 1 audio
    assert float(e[1, 2, 0]) == -2.0 and float(e[1, 5, 0]) == -3.0 and m[1].tolist() == [False, False, True, True, True, True]
    with pytest.raises(ValueError):
        replace_placeholders_and_build_targets(ids, emb, 0, 99, aud[:2], tgt)


def test_lora_starts_as_identity_trains_only_adapters_and_merges():
    torch.manual_seed(0)
    m = CausalLM(LLMConfig(**TINY))
    ids = torch.randint(0, 300, (1, 6))
    before = m(input_ids=ids)["logits"].detach()
    names = apply_lora(m, r=4, lora_alpha=8, target_modules=["q_proj", "v_proj"])
    assert len(names) == 4
    assert torch.allclose(m(input_ids=ids)["logits"], before, atol=1e-6)
    for n, p in m.named_parameters():
        if ".lora_" not in n:
            p.requires_grad_(False)
    trainable = freeze_and_subset(m.named_parameters(), ["^model\\..+$"], [])
    assert trainable and all(".lora_" in n for n, _ in trainable)
    m(input_ids=ids)["logits"].pow(2).mean().backward()
    with torch.no_grad():
        for _, p in trainable:
            p.add_(0.05 * torch.randn_like(p))
    changed = m(input_ids=ids)["logits"].detach()
    merge_lora(m)
    assert torch.allclose(m(input_ids=ids)["logits"], changed, atol=1e-4)
    assert not any(".lora_" in n for n, _ in m.named_parameters())


def test_salm_trains_and_generates():
    torch.manual_seed(0)
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    cfg = OmegaConf.create({
        "audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": dict(TINY, tie_word_embeddings=True),
        "perception": {"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
                       "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}},
        "freeze_params": ["^perception\\.preprocessor\\..+$", "^llm\\..+$"], "prevent_freeze_params": [],
        "train_ds": {"synthetic": {"num_samples": 16}, "batch_size": 4, "shuffle": True},
        "optim": {"name": "adamw", "lr": 3e-3, "weight_decay": 0.0}})
    m = SALM(cfg, tokenizer=tok)
    assert not any(p.requires_grad for n, p in m.named_parameters() if n.startswith("llm."))
    assert m.llm.model.embed_tokens is None and m.embed_tokens.num_embeddings >= tok.vocab_size
    losses = []

    class Rec:
        def on_train_batch_end(self, trainer, model, outputs, batch, batch_idx):
            losses.append(float(outputs["loss"]))

    Trainer(max_steps=12, accelerator="cpu", log_every_n_steps=1, enable_checkpointing=False, logger=False, callbacks=[Rec()]).fit(m)
    assert all(math.isfinite(l) for l in losses) and min(losses[-4:]) < losses[0]
    m.eval()
    out = m.generate([[{"role": "user", "content": "Transcribe: <|audioplaceholder|>"}]] * 2, audios=torch.randn(2, 12000),
                     audio_lens=torch.tensor([12000, 8000]), max_new_tokens=5)
    assert out.shape[0] == 2 and out.shape[1] <= 5


def test_heartbeat_straggler_and_fault_tolerance_on_host(tmp_path):
    now = [1000.0]
    hb0 = HeartbeatMonitor(0, 3, timeout=30.0, directory=str(tmp_path), clock=lambda: now[0])
    hb1 = HeartbeatMonitor(1, 3, timeout=30.0, directory=str(tmp_path), clock=lambda: now[0])
    hb0.beat(1)
    hb1.beat(1)
    assert hb0.dead_ranks() == [2]                    # rank 2 never joined
    now[0] += 60
    hb0.beat(2)
    assert hb0.dead_ranks() == [1, 2]                 # rank 1 stopped beating
    t = [0.0]
    sd = StragglerDetectionCallback(report_time_interval=0.0, clock=lambda: t[0], stop_if_detected=True)

    class Tr:
        callback_metrics = {}
        should_stop = False
        global_rank, world_size, global_step, log_dir = 0, 3, 0, str(tmp_path)

    tr = Tr()
    for dur in (1.0, 1.0, 2.5):
        sd.on_train_batch_start(tr, None, None, 0)
        t[0] += dur
        sd.on_train_batch_end(tr, None, None, None, 0)
    assert sd.last_report["individual_perf"] == pytest.approx(0.4) and tr.callback_metrics["straggler/individual_perf"] < 0.7
    ft = FaultToleranceCallback(heartbeat_timeout=30.0, directory=str(tmp_path / "hb"), exit_on_failure=False, save_on_failure=False)
    ft.setup(tr, None, "fit")
    ft.on_train_batch_end(tr, None, None, None, 0)
    assert tr.should_stop and "no heartbeat from ranks [1, 2]" in ft.failures[0]


def test_packed_sequences_cp_partition_chunking_and_metrics():
    from speech_b200.speechlm import parts

    e = [torch.randn(5, 4), torch.randn(8, 4)]
    t = [torch.arange(5), torch.arange(8)]
    p = parts.pack_sequences(e, t, cp_size=2, tp_size=3)
    assert p.cu_seqlens.tolist() == [0, 4, 12, 12] or p.cu_seqlens.tolist()[-1] % 3 == 0
    assert p.input_embeds.shape[1] == p.target_ids.shape[1] == int(p.cu_seqlens[-1]) and p.input_embeds.shape[1] % 3 == 0
    assert p.target_ids[0, :4].tolist() == [1, 2, 3, 4] and p.position_ids[0, 4:7].tolist() == [0, 1, 2]
    # the packed row attends block-diagonally: logits equal the per-sequence logits
    m = CausalLM(LLMConfig(**TINY)).eval()
    a, b = torch.randn(1, 4, 64), torch.randn(1, 6, 64)
    row = torch.cat([a, b], dim=1)
    seq = torch.tensor([[0] * 4 + [1] * 6])
    pos = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3, 4, 5]])
    packed = m(inputs_embeds=row, position_ids=pos, seq_ids=seq)["logits"]
    assert torch.allclose(packed[:, :4], m(inputs_embeds=a)["logits"], atol=1e-4)
    assert torch.allclose(packed[:, 4:], m(inputs_embeds=b)["logits"], atol=1e-4)
    idx0 = parts.thd_partition_indices(torch.tensor([0, 8, 16]), cp_size=2, cp_rank=0)
    idx1 = parts.thd_partition_indices(torch.tensor([0, 8, 16]), cp_size=2, cp_rank=1)
    assert sorted(idx0.tolist() + idx1.tolist()) == list(range(16)) and idx0.tolist()[:4] == [0, 1, 6, 7]
    aud = torch.randn(2, 1000)
    ch, cl, owner = parts.chunk_audio(aud, torch.tensor([1000, 450]), 400)
    assert ch.shape == (5, 400) and cl.tolist() == [400, 400, 200, 400, 50] and owner.tolist() == [0, 0, 0, 1, 1]
    emb, lens = parts.recombine_chunk_embeddings(torch.ones(5, 3, 2), torch.tensor([3, 3, 2, 3, 1]), owner, 2)
    assert lens.tolist() == [8, 4] and emb.shape == (2, 8, 2)
    a0, l0, real0 = parts.split_audio_for_cp(aud, torch.tensor([1000, 450]), cp_size=4, cp_rank=3)
    assert real0 == 0 and a0.shape == (1, 1000) and l0.tolist() == [1]
    assert parts.bleu(["the cat sat on the mat"], ["the cat sat on the mat"]) == pytest.approx(100.0)
    assert parts.bleu(["a b c d e"], ["v w x y z"]) == 0.0
    lg = torch.zeros(1, 3, 5)
    lg[0, 0, 2] = lg[0, 1, 1] = lg[0, 2, 0] = 5.0
    assert parts.token_accuracy(lg, torch.tensor([[2, 4, -100]])) == 0.5


def test_duplex_models_and_salm_variants():
    from speech_b200.speechlm.duplex import DuplexS2SModel, DuplexSTTModel, SALMWithAsrDecoder
    from speech_b200.speechlm.salm_automodel import SALMAutomodel, pack_sequences

    torch.manual_seed(0)
    pc = {"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}
    cfg = OmegaConf.create({"llm": dict(TINY), "perception": pc, "codebook_size": 10, "num_codebooks": 2, "optim": {"name": "adamw", "lr": 1e-3}})
    audio, lens = torch.randn(2, 16000), torch.tensor([16000, 12000])
    stt = DuplexSTTModel(cfg)
    T = 30
    tgt = torch.randint(3, 50, (2, T))
    loss = stt.training_step({"source_audio": audio, "source_audio_lens": lens, "target_tokens": tgt}, 0)["loss"]
    loss.backward()
    assert math.isfinite(float(loss)) and stt.embed_tokens.weight.grad is not None
    res = stt.offline_inference(audio, lens)
    assert res["tokens"].shape[0] == 2 and res["tokens"].shape[1] == int(res["lengths"].max()) and len(res["text"]) == 2
    # incremental frame-by-frame decoding equals teacher-forced decoding on its own outputs
    inp_prev = torch.cat([torch.full((2, 1), stt.text_pad_id), res["tokens"][:, :-1]], dim=1)
    emb, _ = stt.perception(input_signal=audio, input_signal_length=lens)
    full = stt(stt._frame_inputs(emb, inp_prev))["text_logits"].argmax(-1)
    assert torch.equal(full, res["tokens"])
    s2s = DuplexS2SModel(cfg)
    codes = torch.randint(0, 10, (2, T, 2))
    l = s2s.training_step({"source_audio": audio, "source_audio_lens": lens, "target_tokens": tgt, "target_codes": codes}, 0)["loss"]
    l.backward()
    assert math.isfinite(float(l)) and s2s.audio_head.weight.grad is not None and s2s.speech_vocab_size == 13
    out = s2s.offline_inference(audio, lens, decode_audio=False)
    assert out["codes"].shape == (2, out["tokens"].shape[1], 2) and int(out["codes"].max()) < 13
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    scfg = OmegaConf.create({"audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": dict(TINY, tie_word_embeddings=True), "perception": pc,
                             "freeze_params": [], "prevent_freeze_params": [], "asr_weight": 0.5, "optim": {"name": "adamw", "lr": 1e-3}})
    m = SALMWithAsrDecoder(scfg, tokenizer=tok)
    emb, el = m.perception(input_signal=audio, input_signal_length=lens)
    aux = m.asr_loss(emb, el, torch.randint(5, 200, (2, 6)), torch.tensor([6, 4]))
    aux.backward()
    assert math.isfinite(float(aux)) and m.asr_head.weight.grad is not None
    hyp = m.transcribe_with_asr_head(audio, lens)
    assert len(hyp) == 2 and all(isinstance(h, list) for h in hyp)
    auto = SALMAutomodel(scfg, tokenizer=tok)
    auto.configure_model(None)
    assert auto.device_mesh is None
    # packed rows give the same loss as the padded batch
    from speech_b200.speechlm.data import SALMDataset, synthetic_conversations
    ds = SALMDataset(synthetic_conversations(3, seed=1), tok, auto.prompt_formatter(), scfg.audio_locator_tag, auto.text_pad_id)
    batch = ds.collate([ds[i] for i in range(3)])
    auto.eval()
    ls, n, correct, inp = auto._token_loss_sums(batch)
    pk = pack_sequences(inp["input_embeds"], inp["attention_mask"], inp["target_ids"])
    assert pk["input_embeds"].shape[0] == 1 and int(pk["seq_ids"].max()) == 3 and int((pk["target_ids"] != -100).sum()) == int(n)
    assert int(pk["position_ids"].max()) == int(inp["attention_mask"].sum(1).max()) - 1
    from speech_b200.core.config import open_dict
    with open_dict(auto.cfg):
        auto.cfg.packed_sequences = {"enabled": True, "row_len": None}
    ls2, n2, correct2, _ = auto._token_loss_sums(batch)
    assert int(n2) == int(n) and abs(float(ls2) - float(ls)) < 1e-3 * abs(float(ls)) and int(correct2) == int(correct)
    rows = pack_sequences(inp["input_embeds"], inp["attention_mask"], inp["target_ids"], row_len=int(inp["attention_mask"].sum(1).max()) + 2)
    assert rows["input_embeds"].shape[0] >= 2 and len(rows["cu_seqlens"]) == rows["input_embeds"].shape[0]


def test_ear_tts_mog_rvq_duplex_speech_decoder_and_voice_chat():
    from speech_b200.speechlm.duplex import DuplexSTTModel
    from speech_b200.speechlm.ear_tts import (DuplexEARTTS, DuplexS2SSpeechDecoderModel, EARTTSModel, MoGHead, NemotronVoiceChat,
                                              ResidualVQ)

    torch.manual_seed(0)
    rvq = ResidualVQ(3, 16, 8)
    codes = torch.randint(0, 16, (2, 5, 3))
    lat = rvq.embed(codes)
    assert lat.shape == (2, 5, 8)
    # a latent that is exactly a depth sum quantises to a tuple with the same sum (greedy residual search is consistent)
    again = rvq.embed(rvq.encode(lat))
    assert float((again - lat).norm()) <= float(lat.norm()) * 0.5
    assert torch.allclose(rvq.embed(codes, torch.full((2, 5), 1)), rvq.codebooks[0][codes[..., 0]])
    head = MoGHead(32, 64, 8, num_layers=1, num_predictions=4, low_rank=4)
    x = torch.randn(6, 32)
    logits, mus, logs = head(x)
    assert logits.shape == (6, 4) and mus.shape == (6, 4, 8) and logs.shape == (6, 1)
    # the mixture density integrates to one: NLL of a one-component head equals the Gaussian formula
    one = MoGHead(32, 64, 8, num_layers=1, num_predictions=1, low_rank=None)
    _, mu1, ls1 = one(x)
    tgt = torch.randn(6, 8)
    want = 0.5 * ((tgt - mu1[:, 0]) ** 2).sum(-1) * torch.exp(-2 * ls1[:, 0]) + 8 * ls1[:, 0] + 4 * math.log(2 * math.pi)
    assert torch.allclose(one.nll(x, tgt), want, atol=1e-4)
    g = torch.Generator().manual_seed(1)
    s = head.infer(x, top_p_or_k=1, generator=g)              # top-1: the mean of the most likely component
    best = logits.argmax(-1)
    assert torch.allclose(s, mus[torch.arange(6), best], atol=1e-5)
    cfg = OmegaConf.create({"tts": {"backbone": dict(TINY), "num_quantizers": 3, "codebook_size": 16, "latent_size": 8, "num_predictions": 4,
                                    "low_rank": 4, "cfg_dropout": 0.5}, "optim": {"name": "adamw", "lr": 1e-3}})
    tts = DuplexEARTTS(cfg)
    batch = {"target_tokens": torch.randint(3, 50, (2, 12)), "target_codes": torch.randint(0, 16, (2, 12, 3)), "target_lens": torch.tensor([12, 9])}
    loss = tts.training_step(batch, 0)["loss"]
    loss.backward()
    assert math.isfinite(float(loss)) and tts.tts.head.proj_logits.weight.grad is not None and tts.tts.rvq.codebooks.grad is None
    gen = tts.offline_inference(batch["target_tokens"][:, :6], guidance_scale=1.5, top_p_or_k=2)
    assert gen["codes"].shape == (2, 6, 3) and int(gen["codes"].max()) < 16
    # incremental generation with caches equals the teacher-forced forward on its own outputs (top-1, no noise)
    m: EARTTSModel = tts.tts.eval()
    toks = batch["target_tokens"][:1, :5]
    c = m.generate(toks, top_p_or_k=1)
    hist = m.rvq.embed(c)
    prev = torch.cat([m.bos_emb.expand(1, 1, -1), hist[:, :-1]], dim=1)
    h = m.backbone(inputs_embeds=m._inputs(prev, toks), return_hidden=True)["hidden_states"]
    lg, mu, _ = m.head(h)
    full = m.rvq.encode(mu[0, torch.arange(5), lg[0].argmax(-1)])
    assert torch.equal(full, c[0])
    pc = {"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}
    scfg = OmegaConf.create({"llm": dict(TINY), "perception": pc, "codebook_size": 10, "num_codebooks": 2,
                             "speech_decoder": dict(TINY, num_hidden_layers=1), "optim": {"name": "adamw", "lr": 1e-3}})
    audio, lens = torch.randn(2, 16000), torch.tensor([16000, 12000])
    sd = DuplexS2SSpeechDecoderModel(scfg)
    l = sd.training_step({"source_audio": audio, "source_audio_lens": lens, "target_tokens": torch.randint(3, 50, (2, 30)),
                          "target_codes": torch.randint(0, 10, (2, 30, 2))}, 0)["loss"]
    l.backward()
    assert math.isfinite(float(l)) and sd.audio_head.weight.grad is not None and sd.hidden_proj.weight.grad is not None
    out = sd.offline_inference(audio, lens)
    assert out["codes"].shape == (2, out["tokens"].shape[1], 2) and len(out["text"]) == 2
    chat = NemotronVoiceChat(DuplexSTTModel(scfg), tts)
    res = chat.offline_inference(audio, lens, top_p_or_k=1)
    assert res["codes"].shape[:2] == res["tokens"].shape and res["codes"].shape[2] == 3
    # the speaking half lags the text channel by one frame: the first spoken frame is conditioned on PAD
    st = chat.init_state(2, audio.device)
    assert int(st["pending_text"][0]) == chat.stt.text_pad_id


def test_serving_plugin_token_estimator_lora_merge_export_and_splice(tmp_path):
    from speech_b200.speechlm import vllm_plugin as vp
    from speech_b200.speechlm.perception import AudioPerceptionModule

    torch.manual_seed(0)
    est = vp.AudioTokenEstimator()
    pc = OmegaConf.create({"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
                           "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}, "output_dim": 64})
    perc = AudioPerceptionModule(pc).eval()
    # the integer arithmetic predicts the encoder's real output length
    for n in (1600, 4000, 15999, 16000, 23457, 48000):
        _, ln = perc(input_signal=torch.randn(1, n), input_signal_length=torch.tensor([n]))
        assert est.single_pass(n) == int(ln[0]), n
    # chunking: a short tail is folded into the previous chunk; the total is the sum over chunks
    assert est.spans(68000, 2.0) == [(0, 32000), (32000, 68000)]
    assert est.spans(16000 * 5, 2.0)[-1] == (64000, 80000)
    assert est.tokens(68000, 2.0) == est.single_pass(32000) + est.single_pass(36000)
    for tgt in (7, 100, 333):
        n = est.samples_for_tokens(tgt, 2.0)
        assert est.tokens(n, 2.0) >= tgt and est.tokens(n - 1, 2.0) < tgt
    # LoRA merge
    w, a, b = torch.randn(6, 4), torch.randn(2, 4), torch.randn(6, 2)
    merged = vp.merge_lora_into_base({"l.q.base.weight": w, "l.q.lora_A": a, "l.q.lora_B": b, "l.norm.weight": torch.ones(4)}, 0.5)
    assert set(merged) == {"l.q.weight", "l.norm.weight"} and torch.allclose(merged["l.q.weight"], w + 0.5 * b @ a, atol=1e-6)
    with pytest.raises(KeyError):
        vp.merge_lora_into_base({"x.lora_A": a, "x.lora_B": b}, 1.0)
    # splice
    emb = torch.nn.Embedding(50, 64)
    srv = vp.SpeechLMServingModel(perc, emb, placeholder_id=49, estimator=est, encoder_chunk_size_seconds=1.0)
    audio, lens = torch.randn(2, 40000), torch.tensor([40000, 9000])
    mm = srv.get_multimodal_embeddings(audio, lens)
    assert [m.shape[0] for m in mm] == [est.tokens(40000, 1.0), est.tokens(9000, 1.0)] and mm[0].shape[1] == 64
    ids = srv.expand_placeholders([3, 49, 5, 49, 7], [40000, 9000])
    assert ids.count(49) == mm[0].shape[0] + mm[1].shape[0]
    full = srv.get_input_embeddings(torch.tensor(ids), mm)
    assert full.shape == (len(ids), 64) and torch.allclose(full[1], mm[0][0]) and torch.allclose(full[0], emb.weight[3])
    with pytest.raises(ValueError):
        srv.get_input_embeddings(torch.tensor(ids[:-3] + [1, 1, 1]), mm)
    # registration hands the lazy class path to the engine's registry
    seen = {}

    class _Reg:
        @staticmethod
        def register_model(name, path):
            seen[name] = path

    vp.register(_Reg)
    assert seen == {vp.ARCHITECTURE: "speech_b200.speechlm.vllm_plugin:" + vp.ARCHITECTURE}


def test_sparse_moe_block_matches_per_token_reference_and_per_expert_checkpoints(tmp_path):
    from speech_b200.speechlm.llm import CausalLM, LLMConfig
    from speech_b200.speechlm.moe import SparseMoEBlock, collect_expert_loads, enable_load_tracking, load_balance_summary, moe_aux_loss

    torch.manual_seed(0)
    blk = SparseMoEBlock(16, 24, num_experts=6, top_k=2, norm_topk_prob=True, aux_loss_coef=0.01).train()
    x = torch.randn(3, 5, 16, requires_grad=True)
    y = blk(x)
    # reference: token by token, expert by expert
    xf = x.detach().reshape(-1, 16)
    probs = torch.softmax(xf @ blk.gate.weight.T, -1)
    w, idx = probs.topk(2, -1)
    w = w / w.sum(-1, keepdim=True)
    ref = torch.zeros_like(xf)
    for n in range(xf.shape[0]):
        for j in range(2):
            e = int(idx[n, j])
            g, u = (blk.gate_up[e] @ xf[n]).chunk(2)
            ref[n] += w[n, j] * (blk.down[e] @ (torch.nn.functional.silu(g) * u))
    assert torch.allclose(y.reshape(-1, 16), ref, atol=1e-5)
    aux = moe_aux_loss(blk)
    assert aux is not None and 0.005 < float(aux) < 0.05 and moe_aux_loss(blk) is None
    (y.sum() + aux).backward()
    assert blk.gate.weight.grad is not None and blk.gate_up.grad is not None and x.grad is not None
    # uniform router -> auxiliary loss of exactly coef
    with torch.no_grad():
        blk.gate.weight.zero_()
    p = torch.full((12, 6), 1 / 6)
    assert abs(float(blk.load_balancing_loss(p, torch.arange(24).view(12, 2) % 6)) - 1.0) < 1e-6
    # an LLM with sparse layers; per-expert checkpoint layout round trip
    cfg = LLMConfig(vocab_size=64, hidden_size=16, intermediate_size=32, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=4,
                    num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8, router_aux_loss_coef=0.001, mlp_only_layers=(0,),
                    model_type="qwen3_moe", tie_word_embeddings=False)
    lm = CausalLM(cfg).eval()
    kinds = [type(l.mlp).__name__ for l in lm.model.layers]
    assert kinds == ["MLP", "SparseMoEBlock", "SparseMoEBlock"]
    ids = torch.randint(0, 64, (2, 7))
    out = lm(input_ids=ids)["logits"]
    sd = {k: v for k, v in lm.state_dict().items() if ".mlp.gate_up" not in k and ".mlp.down" not in k or "layers.0." in k}
    for i in (1, 2):
        sd.pop(f"model.layers.{i}.mlp.gate.weight")
        sd.update(lm.model.layers[i].mlp.per_expert_state(prefix=f"model.layers.{i}.mlp."))
    assert "model.layers.1.mlp.experts.3.up_proj.weight" in sd
    import json, os
    from safetensors.torch import save_file
    d = tmp_path / "moe"
    os.makedirs(d)
    save_file({k: v.contiguous() for k, v in sd.items()}, str(d / "model.safetensors"))
    hf = {k: getattr(cfg, k) for k in cfg.__dataclass_fields__}
    hf["mlp_only_layers"] = list(cfg.mlp_only_layers)
    json.dump(hf, open(d / "config.json", "w"))
    lm2 = CausalLM.from_pretrained(str(d)).eval()
    assert torch.allclose(lm2(input_ids=ids)["logits"], out, atol=1e-5)
    enable_load_tracking(lm2)
    lm2(input_ids=ids)
    loads = collect_expert_loads(lm2)
    assert len(loads) == 2 and all(float(v.sum()) == 2 * 7 * 2 for v in loads.values())
    s = load_balance_summary(loads)
    assert s["moe/max_over_mean_load"] >= 1.0 and 0.0 <= s["moe/idle_expert_fraction"] <= 1.0


def test_duplex_stt_streaming_engine_prompts_turn_taking_and_chunked_feeding():
    from speech_b200.speechlm.duplex import DuplexSTTModel
    from speech_b200.speechlm.duplex_streaming import DuplexState, DuplexSTTStreamingInference

    torch.manual_seed(0)
    pc = {"preprocessor": {**preprocessor_cfg(32), "dither": 0.0}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}
    cfg = OmegaConf.create({"llm": dict(TINY), "perception": pc, "predict_user_text": True, "optim": {"name": "adamw", "lr": 1e-3}})
    m = DuplexSTTModel(cfg).eval()
    assert m.predict_user_text
    audio, lens = torch.randn(2, 16000), torch.tensor([16000, 12000])
    # training with both channels
    T = 12
    loss = m.training_step({"source_audio": audio, "source_audio_lens": lens, "target_tokens": torch.randint(3, 50, (2, T)),
                            "source_tokens": torch.randint(3, 50, (2, T))}, 0)["loss"]
    loss.backward()
    assert m.asr_head.weight.grad is not None and m.embed_asr_tokens.weight.grad is not None
    eng = m.streaming_inference
    plain = eng.offline_inference(audio, lens)
    assert plain["tokens"].shape == plain["asr_tokens"].shape and plain["tokens"].shape[1] == int(plain["lengths"].max())
    # the cached frame loop equals teacher forcing on its own outputs
    emb, _ = m.perception(input_signal=audio, input_signal_length=lens)
    prev_t = torch.cat([torch.full((2, 1), m.text_pad_id), plain["tokens"][:, :-1]], 1)
    prev_a = torch.cat([torch.full((2, 1), m.text_pad_id), plain["asr_tokens"][:, :-1]], 1)
    full = m(m._frame_inputs(emb, prev_t, None, prev_a))
    assert torch.equal(full["text_logits"].argmax(-1), plain["tokens"]) and torch.equal(full["asr_logits"].argmax(-1), plain["asr_tokens"])
    # prompts of different lengths are right aligned; trailing padding adds frames
    prompts = torch.tensor([[5, 6, 7], [9, 0, 0]])
    withp = eng.offline_inference(audio, lens, prompt_tokens=prompts, prompt_token_lens=torch.tensor([3, 1]), input_pad_len=3200)
    assert withp["tokens"].shape[1] > plain["tokens"].shape[1]
    # forced turn taking: silence after speech on the user channel forces the agent to start
    st = DuplexState(cache=[dict() for _ in m.llm.model.layers])
    force = DuplexSTTStreamingInference(m, force_turn_taking=True, threshold=6, pad_window=3)
    st.gen_text = [torch.full((1,), m.text_pad_id) for _ in range(5)]
    st.gen_asr = [torch.tensor([11]), torch.tensor([12])] + [torch.full((1,), m.text_pad_id) for _ in range(3)]
    st.t = 5
    out = force._force_turn_taking(st, torch.tensor([33]), torch.tensor([m.text_pad_id]), torch.zeros(1, dtype=torch.bool))
    assert int(out) == m.text_bos_id
    st.gen_text[3] = torch.tensor([m.text_bos_id])         # the agent already started: nothing is forced
    assert int(force._force_turn_taking(st, torch.tensor([33]), torch.tensor([m.text_pad_id]), torch.zeros(1, dtype=torch.bool))) == 33
    st.gen_asr[2:] = [torch.tensor([13]) for _ in range(3)]  # user barges in while the agent talks: agent EOS
    assert int(force._force_turn_taking(st, torch.tensor([33]), torch.tensor([force.user_bos]), torch.zeros(1, dtype=torch.bool))) == m.text_eos_id
    # chunk-by-chunk feeding covers every frame exactly once
    s2 = eng.start(2)
    n = 0
    for k in range(0, 16000, 4000):
        n += eng.feed(s2, audio[:, k:k + 4000])["tokens"].shape[1]
    assert n == s2.t == s2.frames_done and abs(n - plain["tokens"].shape[1]) <= 1


def test_speechlm_metrics_turn_taking_mcq_empty_text_and_results_logger(tmp_path):
    import json
    from speech_b200.speechlm.metrics import (EmptyTextMetric, MCQEvaluator, ResultsLogger, TurnTakingMetrics, compute_turn_taking_metrics,
                                              extract_answer)

    EOS, BOS, PAD = 2, 1, 0
    src = torch.full((4, 40), PAD); prd = torch.full((4, 40), PAD)
    src[0, 10] = EOS; prd[0, 15] = BOS           # 5 frames late: success, 0.4 s
    src[1, 10] = EOS; prd[1, 30] = BOS           # 20 frames late: failure
    src[2, 10] = EOS                             # agent never starts: failure
    prd[3, 5] = BOS                              # user never ends: not counted
    acc, lat = compute_turn_taking_metrics(src, prd, EOS, BOS, tolerance=13, latency_multiplier=0.08)
    assert abs(acc - 1 / 3) < 1e-9 and abs(lat - 0.4) < 1e-9
    tt = TurnTakingMetrics(EOS, BOS)
    tt.update("dev", src, prd); tt.update("dev", src[:1], prd[:1])
    out = tt.compute()
    assert abs(float(out["turn_taking_acc_dev"]) - (1 / 3 + 1) / 2) < 1e-6 and tt.compute() == {}
    cases = {"The answer is B.": "B", "I would choose option (c) because ...": "C", "**D** since the speaker says so": "D", "a": "A",
             "<2> The correct answer is: **A) cats**": "A", "B) the second one": "B", "答案是C": "C", "(d)": "D", "Hard to say, none fits": None, "": None,
             "Looking at the options, (b) is the best answer": "B"}
    for text, want in cases.items():
        assert extract_answer(text) == want, (text, extract_answer(text))
    (tmp_path / "man").mkdir()
    with open(tmp_path / "man" / "quiz.jsonl", "w") as f:
        for i, a in enumerate("ABCD"):
            f.write(json.dumps({"id": f"q{i}", "answer": a}) + "\n")
    ev = MCQEvaluator(str(tmp_path / "man"))
    res = ev.evaluate("quiz", [{"id": "q0", "pred_text": "The answer is A"}, {"id": "q1", "pred_text": "I would pick c"},
                               {"id": "q2", "pred_text": "no idea"}, {"id": "zz", "pred_text": "A"}])
    assert res == {"mcq_acc": 1 / 3, "mcq_answered": 2 / 3, "mcq_total": 3.0}
    em = EmptyTextMetric(); em.update("dev", ["hi", " ", ""]); assert abs(float(em.compute()["empty_text_rate_dev"]) - 2 / 3) < 1e-6
    # two "ranks" write, rank 0 merges (duplicate id from sampler padding is dropped)
    r1 = ResultsLogger(str(tmp_path / "res"), rank=1, world_size=2)
    r1.update("quiz", ["q2", "q0"], ["no idea", "The answer is A"], ["c", "a"])
    r1.reset()
    r0 = ResultsLogger(str(tmp_path / "res"), rank=0, world_size=1, mcq_evaluator=ev)
    r0.world = 2
    r0.update("quiz", ["q0", "q1"], ["The answer is A", "i would pick c"], ["a", "b"])
    m = r0.compute_and_save(["quiz"])
    merged = [json.loads(l) for l in open(tmp_path / "res" / "quiz.jsonl")]
    assert [r["id"] for r in merged] == ["q0", "q1", "q2"] and m["quiz/num_samples"] == 3.0 and m["quiz/mcq_acc"] == 1 / 3
    assert m["quiz/wer"] > 1.0 and m["quiz/empty_text_rate"] == 0.0 and (tmp_path / "res" / "metrics.json").exists()


def test_salm_with_asr_decoder_reads_the_recognisers_hypotheses():
    from speech_b200.models.configs import fastconformer_ctc_config
    from speech_b200.speechlm.data import SALMDataset, synthetic_conversations
    from speech_b200.speechlm.duplex import SALMWithAsrDecoder
    from speech_b200.speechlm.perception import AudioTranscriptionPerceptionModule

    torch.manual_seed(0)
    asr_cfg = OmegaConf.to_container(fastconformer_ctc_config("small", vocab_size=16, dropout=0.0, n_layers=1, features=32, lr=1e-3))
    asr_cfg["preprocessor"]["dither"] = 0.0
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    cfg = OmegaConf.create({"audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": dict(TINY, tie_word_embeddings=True),
                            "perception": {"asr": {"_target_": "speech_b200.models.EncDecCTCModelBPE", **asr_cfg},
                                           "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}},
                            "freeze_params": [], "prevent_freeze_params": [], "asr_weight": 0.0, "asr_transcript_drop_prob": 0.0,
                            "optim": {"name": "adamw", "lr": 1e-3}})
    m = SALMWithAsrDecoder(cfg, tokenizer=tok)
    assert isinstance(m.perception, AudioTranscriptionPerceptionModule) and m.reads_asr_hypotheses
    assert all(not p.requires_grad for p in m.perception.asr.decoder.parameters()) and any(p.requires_grad for p in m.perception.encoder.parameters())
    ds = SALMDataset(synthetic_conversations(2, seed=1), tok, m.prompt_formatter(), cfg.audio_locator_tag, m.text_pad_id)
    batch = ds.collate([ds[0], ds[1]])
    m.eval()
    inp = m.prepare_inputs(batch)
    hyps = m.last_asr_hypotheses
    assert len(hyps) == 2 and all(isinstance(h, str) for h in hyps)
    # sequence length = text tokens - placeholder + audio frames + tokens of ">> hyp <<", per row (left padded to the longest)
    enc, enc_len = m.perception.forward_encoder(batch["audios"], batch["audio_lens"])
    n_text = (batch["input_ids"] != m.text_pad_id).sum(1)
    want = [int(n_text[b]) - 1 + int(enc_len[b]) + len(tok.text_to_ids(m.transcript_template.format(hyps[b]) if hyps[b] else ">> <<")) for b in range(2)]
    assert inp["input_embeds"].shape[1] == max(want) - 1 and inp["attention_mask"].sum(1).tolist() == [w - 1 for w in want]       # left padded; the last position is cut off
    m.train()
    loss = m.training_step(batch, 0)["loss"]
    loss.backward()
    assert math.isfinite(float(loss)) and next(m.perception.encoder.parameters()).grad is not None
    # dropping every hypothesis shortens the inputs
    m.asr_transcript_drop_prob = 1.0
    short = m.prepare_inputs(batch)
    assert short["input_embeds"].shape[1] <= inp["input_embeds"].shape[1] and m.last_asr_hypotheses == ["", ""]


def test_rvq_vae_codec_round_trip_streaming_decode_and_training():
    from speech_b200.speechlm.vae_codec import ProbabilisticRVQ, RVQVAEModel

    torch.manual_seed(0)
    cfg = dict(latent_size=16, n_fft=16, hop_length=4, base_hidden_size=8, channel_mult=(1, 2), rates=(2, 2), num_blocks=1, kernel_size=3,
               codebook_size=32, num_quantizers=3)
    m = RVQVAEModel(cfg).eval()
    assert m.wav_to_token_ratio == 16 and not any(p.requires_grad for p in m.parameters())
    wav = torch.randn(2, 1, 16 * 20) * 0.1
    with pytest.raises(ValueError, match="multiple"):
        m.ae_encode(wav[..., :-3])
    assert m.pad_to_ratio(wav[..., :-3]).shape[-1] == 320
    ids = m.encode(wav)
    assert len(ids) == 3 and ids[0].shape == (2, 20) and int(ids[0].max()) < 32
    full = m.decode(ids)
    assert full.shape == (2, 1, 320) and float(full.abs().max()) <= 1.0
    # residual quantisation: every level lowers the error
    z = m.ae_encode(wav)
    errs = [float((z - m.prvq.decode(ids[: k + 1])).pow(2).mean()) for k in range(3)]
    assert errs[0] >= errs[1] >= errs[2]
    # causal: decode in chunks of latents equals the one-shot decode; later latents do not change earlier samples
    zq = m.prvq.decode(ids)
    state, outs = None, []
    for a, b in ((0, 7), (7, 8), (8, 20)):
        y, state = m.decode_stream(zq[:, a:b], state)
        outs.append(y)
    assert torch.allclose(torch.cat(outs, -1), full, atol=1e-5)
    z2 = zq.clone()
    z2[:, 12:] += 1.0
    assert torch.allclose(m.ae_decode(z2)[..., : 12 * 16], full[..., : 12 * 16], atol=1e-6)
    # training: reconstruction improves, codebooks move toward the latents, variance tracks the residual
    t = RVQVAEModel(cfg, trainable=True).train()
    sig = torch.sin(torch.arange(320) * 0.2)[None, None].repeat(2, 1, 1) * 0.5
    opt = torch.optim.Adam([p for p in t.parameters() if p.requires_grad], 3e-3)
    v0 = t.prvq.variance.clone()
    first = None
    for _ in range(40):
        opt.zero_grad()
        out = t.training_loss(sig)
        out["loss"].backward()
        opt.step()
        first = first if first is not None else float(out["loss"])
    assert float(out["loss"]) < 0.7 * first and not torch.equal(t.prvq.variance, v0)
    assert float(ProbabilisticRVQ(8, 4, 2).log_std) == 0.0
    audio, alen = m.decode(tokens=torch.stack(ids, dim=1), tokens_len=torch.tensor([20, 10]))
    assert torch.allclose(audio, full[:, 0]) and alen.tolist() == [320, 160] and m.rvq_codebooks.shape == (3, 32, 16)


def test_duplex_token_channels_dataset_augmenter_and_chunked_perception():
    from speech_b200.speechlm.duplex_data import (AudioAugmenter, DuplexConversationDataset, build_token_channel, configure_optimizers_exclude_norm_from_wd,
                                                  delay_eos, encode_audio_with_optional_chunking, synthetic_duplex_conversations, text_with_timestamps_to_ids,
                                                  tokens_to_str)

    class Tok:
        def text_to_ids(self, t):
            return [10 + "abcdefgh".index(c) for c in t.replace(" ", "")]

        def ids_to_text(self, ids):
            return "".join("abcdefgh"[i - 10] for i in ids)

    tok = Tok()
    turns = [{"role": "user", "start": 0.0, "end": 0.8, "text": "ab"}, {"role": "agent", "start": 1.0, "end": 1.6, "text": "cde"},
             {"role": "agent", "start": 2.0, "end": 2.3, "text": "fgh"}]
    ch = build_token_channel(turns, {"agent"}, tok, 0.1, 30, bos_id=1, eos_id=2, pad_id=0)
    assert ch[10:17].tolist() == [1, 12, 13, 14, 0, 0, 2] and ch[20:24].tolist() == [1, 15, 16, 2]          # the last turn is cut to fit before its end
    usr = build_token_channel(turns, {"user"}, tok, 0.1, 30, 1, 2, 0)
    assert usr[:9].tolist() == [1, 10, 11, 0, 0, 0, 0, 0, 2] and int(usr[9:].sum()) == 0
    assert text_with_timestamps_to_ids("<|0.0|> a <|0.5|> bc", tok, 0.1) == [(0, [10]), (5, [11, 12])]
    timed = build_token_channel([{"role": "agent", "start": 1.0, "end": 2.0, "text": "<|0.0|> a <|0.5|> bc"}], {"agent"}, tok, 0.1, 30, 1, 2, 0)
    assert timed[10:21].tolist() == [1, 10, 0, 0, 0, 0, 11, 12, 0, 0, 2]
    d = delay_eos(torch.tensor([[1, 5, 2, 0, 0, 0, 1, 6, 2, 0]]), 2, 0, shift=2)
    assert d.tolist() == [[1, 5, 0, 0, 2, 0, 1, 6, 0, 2]]
    assert tokens_to_str(torch.tensor([[1, 10, 11, 0, 2, 0]]), torch.tensor([6]), tok, 0, True, 1, 2) == ["<bos> ab <eos>"]
    assert tokens_to_str(torch.tensor([[1, 10, 11, 0, 2, 0]]), torch.tensor([6]), tok, 0, False, 1, 2) == ["ab"]
    ds = DuplexConversationDataset(synthetic_duplex_conversations(3, num_codebooks=2, duration=1.0), tok, frame_sec=0.08, eos_delay=1)
    b = ds.collate_fn([ds[0], ds[1]])
    assert b["source_audio"].shape == (2, 16000) and b["target_tokens"].shape == (2, 13) and b["target_codes"].shape == (2, 13, 2) and b["token_lens"].tolist() == [13, 13]
    assert int((b["target_tokens"] == 1).sum()) == 2 and int((b["source_tokens"] == 1).sum()) == 2
    x = torch.sin(torch.arange(16000) * 0.3) * 0.5
    aug = AudioAugmenter(noise_prob=1.0, snr_range=(10, 10), gain_prob=0.0, lowpass_prob=0.0)
    y = aug(x, 16000)
    assert 10 * torch.log10(x.pow(2).mean() / (y - x).pow(2).mean()) == pytest.approx(10.0, abs=0.3)
    lp = AudioAugmenter(lowpass_prob=1.0, lowpass_hz_range=(2000, 2000))(x + torch.sin(torch.arange(16000) * 2.5) * 0.5, 16000)
    spec = torch.fft.rfft(lp).abs()
    assert spec[int(0.3 / (2 * math.pi) * 16000)] > 50 * spec[int(2.5 / (2 * math.pi) * 16000)]               # 764 Hz passes, 6.4 kHz is removed

    class Perc(torch.nn.Module):
        calls = []

        def forward(self, input_signal, input_signal_length):
            Perc.calls.append(tuple(input_signal.shape))
            e = input_signal.unfold(1, 160, 160).mean(-1, keepdim=True).repeat(1, 1, 4)
            return e, input_signal_length // 160

    audio, lens = torch.randn(2, 16000), torch.tensor([16000, 9000])
    whole, wl = encode_audio_with_optional_chunking(Perc(), audio, lens)
    parts, pl = encode_audio_with_optional_chunking(Perc(), audio, lens, chunk_size_seconds=0.25, min_chunk_seconds=0.1)
    assert Perc.calls[-1] == (6, 5000) and pl.tolist() == wl.tolist() == [100, 56] and torch.allclose(parts[1, :56], whole[1, :56], atol=1e-6)
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4))
    opt = configure_optimizers_exclude_norm_from_wd(net, lr=1e-3, weight_decay=0.1)
    assert [len(g["params"]) for g in opt.param_groups] == [1, 3] and [g["weight_decay"] for g in opt.param_groups] == [0.1, 0.0]


def test_duplex_models_train_from_their_config_data_blocks():
    from speech_b200.core.trainer import Trainer
    from speech_b200.speechlm.duplex import DuplexS2SModel, DuplexSTTModel

    torch.manual_seed(0)
    base = {"llm": {"vocab_size": 64, "hidden_size": 32, "intermediate_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4, "num_key_value_heads": 2,
                    "head_dim": 8}, "predict_user_text": True,
            "perception": {"preprocessor": {"_target_": "speech_b200.modules.preprocessor.AudioToMelSpectrogramPreprocessor", "features": 16, "dither": 0.0},
                           "encoder": {"_target_": "speech_b200.modules.conformer_encoder.ConformerEncoder", "feat_in": 16, "n_layers": 1, "d_model": 32,
                                       "subsampling": "dw_striding", "subsampling_factor": 8, "subsampling_conv_channels": 16, "n_heads": 4},
                           "modality_adapter": {"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 32}},
            "train_ds": {"synthetic": {"num_samples": 4, "duration": 1.0}, "batch_size": 2}, "optim": {"name": "adamw", "lr": 1e-3}}
    for cls, extra in ((DuplexSTTModel, {}), (DuplexS2SModel, {"num_codebooks": 2, "codebook_size": 16})):
        m = cls(OmegaConf.create(dict(base, **extra)))
        assert m._train_dl is not None
        batch = next(iter(m._train_dl))
        assert ("target_codes" in batch) == (cls is DuplexS2SModel)
        tr = Trainer(max_steps=2, accelerator="cpu", devices=1, enable_checkpointing=False, logger=False)
        tr.fit(m)
        assert tr.global_step == 2


def test_speechlm_initialisation_from_checkpoints_of_several_kinds(tmp_path):
    from safetensors.torch import save_file

    from speech_b200.speechlm.pretrained import (init_from_training_checkpoint, init_model_from_checkpoint, init_perception_from_checkpoint, load_checkpoint,
                                                 set_model_dict_for_partial_init)
    from speech_b200.utils.dcp_io import DCPCheckpointIO

    class Perc(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.encoder = torch.nn.Linear(4, 4)
            self.proj = torch.nn.Linear(4, 6)

    class LM(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.perception, self.llm = Perc(), torch.nn.Linear(6, 6)

    torch.manual_seed(0)
    a, b = LM(), LM()
    sd = {k: v.clone() for k, v in a.state_dict().items()}
    save_file(sd, str(tmp_path / "m.safetensors"))
    torch.save({"state_dict": sd, "global_step": 3}, tmp_path / "m.ckpt")
    os.makedirs(tmp_path / "hf")
    keys = sorted(sd)
    save_file({k: sd[k] for k in keys[:3]}, str(tmp_path / "hf" / "model-00001-of-00002.safetensors"))
    save_file({k: sd[k] for k in keys[3:]}, str(tmp_path / "hf" / "model-00002-of-00002.safetensors"))
    DCPCheckpointIO().save_checkpoint(sd, str(tmp_path / "dcp"))
    for p in ("m.safetensors", "m.ckpt", "hf", "dcp"):
        got = load_checkpoint(str(tmp_path / p))
        assert set(got) == set(sd) and torch.equal(got["llm.weight"], sd["llm.weight"]), p
    n_ok, n_skip = init_model_from_checkpoint(b, str(tmp_path / "m.safetensors"))
    assert (n_ok, n_skip) == (6, 0) and torch.equal(b.llm.weight, a.llm.weight)
    # an ASR-style checkpoint: encoder.* goes under perception., the rest is ignored
    c = LM()
    asr_sd = {"encoder.weight": torch.full((4, 4), 2.0), "encoder.bias": torch.zeros(4), "decoder.weight": torch.zeros(9, 4)}
    torch.save(asr_sd, tmp_path / "asr.pt")
    assert init_perception_from_checkpoint(c, str(tmp_path / "asr.pt")) == 2 and float(c.perception.encoder.weight[0, 0]) == 2.0
    assert init_perception_from_checkpoint(c, str(tmp_path / "m.ckpt")) == 4 and torch.equal(c.perception.proj.weight, a.perception.proj.weight)
    torch.save({"x": torch.zeros(1)}, tmp_path / "nothing.pt")
    with pytest.raises(RuntimeError):
        init_perception_from_checkpoint(c, str(tmp_path / "nothing.pt"))
    _, taken, skipped = set_model_dict_for_partial_init({"model.llm.weight": torch.zeros(6, 6), "model.llm.bias": torch.zeros(5)}, b.state_dict(), strip_prefix="model.")
    assert taken == ["llm.weight"] and "shape" in skipped[0]
    assert init_from_training_checkpoint(LM(), str(tmp_path / "dcp")) == 6
    with pytest.raises(RuntimeError):
        init_from_training_checkpoint(torch.nn.Linear(2, 2), str(tmp_path / "m.ckpt"))
