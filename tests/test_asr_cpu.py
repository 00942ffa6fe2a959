"""CPU end-to-end tests: FastConformer-CTC / TDT training, .nemo round trip, decoding, gloo data parallelism."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from speech_b200.core.config import OmegaConf, open_dict
from speech_b200.core.trainer import Trainer
from speech_b200.models import EncDecCTCModelBPE, EncDecHybridRNNTCTCBPEModel, EncDecRNNTBPEModel
from speech_b200.models.configs import fastconformer_ctc_config, fastconformer_transducer_config

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ctc_cfg(n_layers=2, samples=16):
    cfg = fastconformer_ctc_config("small", vocab_size=128, n_layers=n_layers)
    with open_dict(cfg):
        cfg.train_ds = {"synthetic": {"num_samples": samples, "vocab_size": 128, "min_duration": 1.0, "max_duration": 2.0,
                                      "max_tokens_frac_of_frames": 0.5, "token_low": 0}, "batch_size": 4, "shuffle": True}
    return cfg


def test_ctc_trains_and_nemo_roundtrip(tmp_path):
    torch.manual_seed(0)
    model = EncDecCTCModelBPE(_ctc_cfg())
    losses = []

    class Rec:
        def setup(self, *a): ...

        def on_train_batch_end(self, trainer, m, out, batch, idx):
            losses.append(float(out["loss"]))

    tr = Trainer(max_steps=10, accelerator="cpu", callbacks=[Rec()], log_every_n_steps=1)
    tr.fit(model)
    assert all(l == l and l < 1e4 for l in losses)
    assert min(losses[-3:]) < losses[0]
    path = str(tmp_path / "m.nemo")
    model.save_to(path)
    import tarfile

    with tarfile.open(path, "r:") as tar:
        names = sorted(os.path.basename(n) for n in tar.getnames() if n not in (".",))
    assert "model_config.yaml" in names and "model_weights.ckpt" in names
    restored = EncDecCTCModelBPE.restore_from(path, map_location="cpu")
    sd1, sd2 = model.state_dict(), restored.state_dict()
    assert sd1.keys() == sd2.keys()
    assert all(torch.equal(sd1[k], sd2[k]) for k in sd1)
    for key in ("preprocessor.featurizer.window", "preprocessor.featurizer.fb", "encoder.pre_encode.conv.0.weight",
                "encoder.pre_encode.conv.2.weight", "encoder.pre_encode.conv.3.weight", "encoder.pre_encode.out.weight",
                "encoder.layers.0.norm_feed_forward1.weight", "encoder.layers.0.feed_forward1.linear1.weight",
                "encoder.layers.0.self_attn.linear_q.weight", "encoder.layers.0.self_attn.linear_pos.weight",
                "encoder.layers.0.self_attn.pos_bias_u", "encoder.layers.0.conv.pointwise_conv1.weight",
                "encoder.layers.0.conv.depthwise_conv.weight", "encoder.layers.0.conv.batch_norm.running_mean",
                "encoder.layers.0.conv.pointwise_conv2.weight", "encoder.layers.0.norm_out.weight",
                "decoder.decoder_layers.0.weight"):
        assert key in sd1, key
    x = torch.randn(2, 16000) * 0.1
    assert model.transcribe([x[0], x[1]], batch_size=2) == restored.transcribe([x[0], x[1]], batch_size=2)
    cfg_only = EncDecCTCModelBPE.restore_from(path, return_config=True)
    assert cfg_only.encoder.d_model == 176


def test_tdt_and_hybrid_train_and_decode():
    torch.manual_seed(0)
    cfg = fastconformer_transducer_config("small", vocab_size=32, n_layers=1, dropout=0.0, lr=2e-3, sched=None,
                                          hybrid_ctc_weight=0.3)
    with open_dict(cfg):
        cfg.train_ds = {"synthetic": {"num_samples": 8, "vocab_size": 32, "min_duration": 1.0, "max_duration": 1.5,
                                      "tokens_per_second": 3.0}, "batch_size": 4, "shuffle": False}
    model = EncDecHybridRNNTCTCBPEModel(cfg)
    assert "decoder.prediction.embed.weight" in model.state_dict()
    assert "decoder.prediction.dec_rnn.lstm.weight_ih_l0" in model.state_dict()
    assert "joint.joint_net.1.weight" in model.state_dict() and "ctc_decoder.decoder_layers.0.weight" in model.state_dict()
    assert model.joint.num_classes_with_blank == 32 + 1 + 5
    tr = Trainer(max_steps=4, accelerator="cpu", log_every_n_steps=1)
    tr.fit(model)
    assert float(tr.callback_metrics["train_loss"]) == float(tr.callback_metrics["train_loss"])
    x = torch.randn(12000) * 0.1
    hyp = model.transcribe([x], batch_size=1, return_hypotheses=True)[0]
    assert hyp.text is not None and len(hyp.y_sequence) == len(hyp.timestamp)
    model.change_decoding_strategy(decoder_type="ctc")
    assert isinstance(model.transcribe([x], batch_size=1)[0], str)
    model.change_decoding_strategy(OmegaConf.create({"strategy": "beam", "beam": {"beam_size": 2}}), decoder_type="rnnt")
    assert isinstance(model.transcribe([x], batch_size=1)[0], str)


def test_rnnt_plain_and_fused_losses_agree():
    torch.manual_seed(0)
    cfg = fastconformer_transducer_config("small", vocab_size=16, n_layers=1, dropout=0.0, loss="rnnt", lr=1e-3, sched=None)
    m = EncDecRNNTBPEModel(cfg)
    m.eval()
    B, T, U = 2, 8, 3
    enc = torch.randn(B, m.encoder._feat_out, T)
    dec = torch.randn(B, cfg.decoder.prednet.pred_hidden, U + 1)
    tgt = torch.randint(0, 16, (B, U))
    el, tl = torch.tensor([8, 6]), torch.tensor([3, 2])
    fused, *_ = m.joint(encoder_outputs=enc, decoder_outputs=dec, encoder_lengths=el, transcripts=tgt, transcript_lengths=tl)
    m.joint.set_fuse_loss_wer(False)
    logits = m.joint(encoder_outputs=enc, decoder_outputs=dec)
    plain = m.loss(log_probs=logits, targets=tgt, input_lengths=el, target_lengths=tl)
    assert torch.allclose(fused, plain, atol=1e-4)
    ref = torch.nn.functional.ctc_loss  # noqa: F841  (only to make sure torch is importable in spawned ranks)


DDP_SCRIPT = textwrap.dedent("""
    import os, sys, json, torch
    sys.path.insert(0, {repo!r})
    from speech_b200.core.config import open_dict
    from speech_b200.core.trainer import Trainer
    from speech_b200.models import EncDecCTCModelBPE
    from speech_b200.models.configs import fastconformer_ctc_config
    torch.manual_seed(int(os.environ["RANK"]) + 5)   # different init per rank: the broadcast must equalise them
    cfg = fastconformer_ctc_config("small", vocab_size=128, n_layers=1)
    with open_dict(cfg):
        cfg.train_ds = {{"synthetic": {{"num_samples": 32, "vocab_size": 128, "min_duration": 1.0, "max_duration": 2.0,
                                        "max_tokens_frac_of_frames": 0.5}}, "batch_size": 4, "shuffle": True}}
    m = EncDecCTCModelBPE(cfg)
    tr = Trainer(max_steps=3, accelerator="cpu", log_every_n_steps=1)
    tr.fit(m)
    flat = torch.cat([p.detach().flatten() for p in m.parameters()])
    print("RESULT", json.dumps({{"rank": tr.global_rank, "sum": float(flat.double().sum()), "loss": float(tr.callback_metrics["train_loss"])}}))
""")


def test_gloo_data_parallel_keeps_ranks_in_sync(tmp_path):
    script = tmp_path / "ddp.py"
    script.write_text(DDP_SCRIPT.format(repo=REPO))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr[-3000:]
    import json

    res = [json.loads(l.split("RESULT", 1)[1]) for l in out.stdout.splitlines() if "RESULT" in l]
    assert len(res) == 2
    assert abs(res[0]["sum"] - res[1]["sum"]) < 1e-6 * max(1.0, abs(res[0]["sum"]))
    assert res[0]["loss"] != res[1]["loss"]  # each rank saw its own shard of the data


def test_graph_rnnt_and_w_transducer_losses_match_explicit_lattice_dp():
    import math as _m

    from speech_b200.losses.graph_transducer import GraphRnntLoss, GraphWTransducerLoss
    from speech_b200.ops import reference

    torch.manual_seed(0)
    B, T, U, V = 3, 7, 4, 6
    blank = V - 1
    logits = torch.randn(B, T, U + 1, V, dtype=torch.float64, requires_grad=True)
    labels = torch.randint(0, V - 1, (B, U))
    act_lens, label_lens = torch.tensor([7, 5, 6]), torch.tensor([4, 2, 3])
    loss = GraphRnntLoss(blank, double_scores=True)(logits, labels, act_lens, label_lens)
    ref = reference.tdt_loss_from_logits(logits.detach().float(), labels, act_lens, label_lens, blank, [], 0.0)
    assert torch.allclose(loss, ref.float(), atol=1e-3)
    loss.sum().backward()
    assert torch.isfinite(logits.grad).all() and float(logits.grad[1, 5:].abs().sum()) == 0.0     # frames past the length carry no gradient

    def lattice(lp, y, Tn, Un, eps, mode):
        """Plain-Python forward algorithm over the W-Transducer grid with explicit skip arcs."""
        NEG = -1e30
        lae = lambda a, b: max(a, b) + _m.log1p(_m.exp(-abs(a - b))) if min(a, b) > NEG / 2 else max(a, b)  # noqa: E731
        al = [[NEG] * (Un + 1) for _ in range(Tn)]
        for t in range(Tn):
            for u in range(Un + 1):
                s = 0.0 if (t == 0 and u == 0) else NEG
                if t > 0 and u == 0 and eps is not None:
                    s = lae(s, eps)                                   # start state -> (t, 0)
                if t > 0:
                    s = lae(s, al[t - 1][u] + lp[t - 1][u][blank])
                if u > 0:
                    s = lae(s, al[t][u - 1] + lp[t][u - 1][y[u - 1]])
                al[t][u] = s
        end = al[Tn - 1][Un]
        skipped = NEG
        if eps is not None:
            for t in range(Tn - 1):
                skipped = lae(skipped, al[t][Un] + eps)               # (t, U) -> last frame
        if mode == "force_final":
            return lae(end, skipped) + lp[Tn - 1][Un][blank]
        return lae(end + lp[Tn - 1][Un][blank], skipped)

    lp = torch.log_softmax(logits.detach(), -1).tolist()
    for mode in ("force_final", "allow_ignore"):
        for eps in (0.0, -1.5):
            got = GraphWTransducerLoss(blank, eps_weight=eps, last_blank_mode=mode, double_scores=True)(logits, labels, act_lens, label_lens)
            exp = [-lattice(lp[b], labels[b].tolist(), int(act_lens[b]), int(label_lens[b]), eps, mode) for b in range(B)]
            assert torch.allclose(got.double(), torch.tensor(exp, dtype=torch.float64), atol=1e-4), (mode, eps, got, exp)
            assert (got <= loss.detach() + 1e-5).all()                # extra paths can only raise the likelihood
    from speech_b200.losses.rnnt import RNNTLoss

    via = RNNTLoss(num_classes=blank, loss_name="graph_w_transducer", loss_kwargs={"eps_weight": -1.5, "last_blank_mode": "force_final"},
                   reduction="none")
    v = via(log_probs=logits.detach().float(), targets=labels, input_lengths=act_lens, target_lengths=label_lens)
    exp = [-lattice(lp[b], labels[b].tolist(), int(act_lens[b]), int(label_lens[b]), -1.5, "force_final") for b in range(B)]
    assert torch.allclose(v, torch.tensor(exp, dtype=torch.float32), atol=1e-3)


def test_normalised_lstm_variants_thread_state():
    from speech_b200.modules.rnnt import BNRNNSum, LayerNormLSTM, rnn

    torch.manual_seed(0)
    for norm, cls in (("batch", BNRNNSum), ("layer", LayerNormLSTM)):
        m = rnn(16, 24, 2, norm=norm, dropout=0.0, norm_first_rnn=True).eval()
        assert isinstance(m, cls)
        x = torch.randn(7, 3, 16)
        y, (h, c) = m(x)
        y1, st = m(x[:4])
        y2, _ = m(x[4:], st)
        assert y.shape == (7, 3, 24) and h.shape == c.shape == (2, 3, 24)
        assert torch.allclose(torch.cat([y1, y2]), y, atol=1e-6)
        y.sum().backward()
    with pytest.raises(ValueError):
        rnn(16, 24, 1, norm="instance")


def test_subsampling_prime_shapes_leaves_no_gradients_and_keeps_mode():
    import torch

    from speech_b200.modules.subsampling import ConvSubsampling

    sub = ConvSubsampling(subsampling="dw_striding", subsampling_factor=8, feat_in=16, feat_out=32, conv_channels=8).eval()
    before = [p.detach().clone() for p in sub.parameters()]
    sub.prime_shapes([(2, 40), (3, 57)], "cpu")
    assert not sub.training and all(p.grad is None for p in sub.parameters())
    assert all(torch.equal(a, b) for a, b in zip(before, sub.parameters()))


def test_longformer_attention_is_banded_and_matches_dense_masked_attention():
    """Sliding-window relative-position attention computed block by block (no [T, T] tensor) equals dense attention with a
    band mask, for several block sizes, with padding; and it runs on a sequence whose dense score matrix would not fit a test."""
    import torch
    from speech_b200.modules.attention import LocalAttRelPositionalEncoding, RelPositionMultiHeadAttentionLongformer

    torch.manual_seed(0)
    B, T, D, H, left, right = 2, 75, 32, 4, 6, 4
    att = RelPositionMultiHeadAttentionLongformer(H, D, 0.0, att_context_size=(left, right), query_block=16).eval()
    torch.nn.init.normal_(att.pos_bias_u, std=0.3); torch.nn.init.normal_(att.pos_bias_v, std=0.3)
    pe = LocalAttRelPositionalEncoding(att_context_size=[left, right], d_model=D, dropout_rate=0.0)
    pe.extend_pe(T, torch.device("cpu"), torch.float32)
    x = torch.randn(B, T, D)
    _, pos = pe(x)
    pad = torch.zeros(B, T, dtype=torch.bool); pad[1, 60:] = True
    out = att(x, x, x, pad_mask=pad, pos_emb=pos)
    # dense reference
    q, k, v = att._qkv(x, x, x)
    p = torch.nn.functional.linear(pos, att.linear_pos.weight).view(1, -1, H, D // H)
    qu = (q + att.pos_bias_u).transpose(1, 2); qv = (q + att.pos_bias_v).transpose(1, 2)
    ac = qu @ k.transpose(1, 2).transpose(-2, -1)
    bdw = qv @ p.transpose(1, 2).transpose(-2, -1)
    i = torch.arange(T)[:, None]; j = torch.arange(T)[None, :]
    rel = i - j
    band = (rel <= left) & (rel >= -right)
    bd = torch.gather(bdw, 3, (left - rel).clamp(0, left + right)[None, None].expand(B, H, T, T))
    hidden = (~band)[None] | pad[:, None, :] | pad[:, :, None]
    sc = ((ac + bd) / att.s_d_k).masked_fill(hidden[:, None], -10000.0)
    a = torch.softmax(sc, -1).masked_fill(hidden[:, None], 0.0)
    ref = torch.nn.functional.linear((a @ v.transpose(1, 2)).transpose(1, 2).reshape(B, T, D), att.linear_out.weight, att.linear_out.bias)
    assert torch.allclose(out[~pad], ref[~pad], atol=1e-5), (out - ref).abs().max()
    for qb in (1, 7, 200):
        att.query_block = qb
        assert torch.allclose(att(x, x, x, pad_mask=pad, pos_emb=pos)[~pad], ref[~pad], atol=1e-5)
    # global tokens: every frame additionally sees frames 0 and 8; those two see everything
    att2 = RelPositionMultiHeadAttentionLongformer(H, D, 0.0, att_context_size=(left, right), global_tokens=2, global_tokens_spacing=8,
                                                   query_block=16).eval()
    att2.load_state_dict(att.state_dict())
    o2 = att2(x, x, x, pad_mask=pad, pos_emb=pos)
    assert torch.isfinite(o2).all() and not torch.allclose(o2[0, 40], out[0, 40])
    # a long input: 20 000 frames would need 4 x 20000^2 x 4 B = 6.4 GB per batch element as dense scores
    Tl = 20000
    pe.extend_pe(Tl, torch.device("cpu"), torch.float32)
    xl = torch.randn(1, Tl, D)
    _, posl = pe(xl)
    att.query_block = 1024
    assert att(xl, xl, xl, pos_emb=posl).shape == (1, Tl, D)


def test_subsampling_conv_chunking_by_batch_and_by_time_equals_unsplit():
    import torch
    from speech_b200.modules.subsampling import ConvSubsampling

    torch.manual_seed(0)
    for kind in ("dw_striding", "striding"):
        sub = ConvSubsampling(kind, 8, 80, 32, 16, subsampling_conv_chunking_factor=-1).eval()
        x = torch.randn(3, 203, 80)
        lens = torch.tensor([203, 150, 77])
        with torch.no_grad():
            ref, ref_len = sub(x, lens)
            sub.subsampling_conv_chunking_factor = 1
            same, _ = sub(x, lens)                       # far below the 2**31 limit: one piece
            assert torch.equal(same, ref)
            sub.subsampling_conv_chunking_factor = 3     # by batch
            by_batch, l1 = sub(x, lens)
            assert torch.allclose(by_batch, ref, atol=1e-6) and torch.equal(l1, ref_len)
            sub.subsampling_conv_chunking_factor = 16    # a single recording no longer fits: time chunks with halos
            calls = []
            orig = sub._forward_once
            sub._forward_once = lambda a, b: (calls.append(a.shape), orig(a, b))[1]
            by_time, l2 = sub(x, lens)
            assert len(calls) > 3 and max(c[1] for c in calls) < 120
        assert by_time.shape == ref.shape and torch.equal(l2, ref_len)
        for b in range(3):
            n = int(ref_len[b])
            assert torch.allclose(by_time[b, :n], ref[b, :n], atol=1e-5), (kind, b, (by_time[b, :n] - ref[b, :n]).abs().max())


def test_model_level_adapters_strategies_save_load_and_restore(tmp_path):
    import torch
    from speech_b200.core.adapters import (MultiHeadAttentionAdapter, PositionalEncodingAdapter, RelPositionMultiHeadAttentionAdapter,
                                          ResidualAddAdapterStrategy, adapter_auxiliary_loss)
    from speech_b200.models import EncDecCTCModelBPE
    from speech_b200.models.configs import fastconformer_ctc_config

    torch.manual_seed(0)
    m = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=16, dropout=0.0, n_layers=2, lr=1e-3))
    audio, lens = torch.randn(2, 8000), torch.tensor([8000, 6000])
    m.eval()
    base = m.forward(input_signal=audio, input_signal_length=lens)[0]
    m.add_adapter("lin", {"in_features": 176, "dim": 8, "adapter_strategy": {"_target_": "ResidualAddAdapterStrategy", "l2_lambda": 0.1}})
    m.add_adapter("encoder:att", {"_target_": "speech_b200.core.adapters.RelPositionMultiHeadAttentionAdapter", "n_head": 4, "n_feat": 176})
    m.add_adapter("decoder:dec", {"in_features": 176, "dim": 4})
    assert m.get_enabled_adapters() == ["encoder:lin", "encoder:att", "decoder:dec"] and set(m.cfg.adapters.keys()) == {"encoder:lin", "encoder:att", "decoder:dec"}
    # zero-initialised outputs: adding adapters does not change the model
    assert torch.allclose(m.forward(input_signal=audio, input_signal_length=lens)[0], base, atol=1e-5)
    n_train = m.freeze_base_and_train_adapters()
    assert 0 < n_train < 0.3 * sum(p.numel() for p in m.parameters())
    assert all(("adapter_layer" in n) == p.requires_grad for n, p in m.named_parameters())
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "adapter_layer" in n:
                p.add_(0.05 * torch.randn_like(p))
    m.train()
    out = m.forward(input_signal=audio, input_signal_length=lens)[0]
    aux = adapter_auxiliary_loss(m)
    assert aux is not None and float(aux) > 0 and adapter_auxiliary_loss(m) is None
    (out.float().pow(2).mean() + aux).backward()
    assert m.encoder.layers[0].adapter_layer["lin"].module[1].weight.grad is not None
    m.eval()
    with_ad = m.forward(input_signal=audio, input_signal_length=lens)[0]
    m.set_enabled_adapters(enabled=False)
    base = m.forward(input_signal=audio, input_signal_length=lens)[0]        # the training pass above moved the BatchNorm statistics
    assert m.get_enabled_adapters() == [] and not torch.allclose(with_ad, base, atol=1e-4)
    m.set_enabled_adapters("encoder:lin", True)
    only_lin = m.forward(input_signal=audio, input_signal_length=lens)[0]
    m.set_enabled_adapters(enabled=True)
    # adapters alone: save, load into a fresh base model
    m.save_adapters(str(tmp_path / "ad.pt"))
    m.save_adapters(str(tmp_path / "lin.pt"), name="lin")
    assert (tmp_path / "ad.pt").stat().st_size < 0.5 * sum(p.numel() * 4 for p in m.parameters())
    torch.manual_seed(0)
    fresh = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=16, dropout=0.0, n_layers=2, lr=1e-3)).eval()
    base_sd = {k: v for k, v in m.state_dict().items() if "adapter_layer" not in k}     # same base model (BatchNorm statistics included)
    fresh.load_state_dict(base_sd, strict=False)
    fresh.load_adapters(str(tmp_path / "ad.pt"))
    assert torch.allclose(fresh.forward(input_signal=audio, input_signal_length=lens)[0], with_ad, atol=1e-5)
    torch.manual_seed(0)
    fresh2 = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=16, dropout=0.0, n_layers=2, lr=1e-3)).eval()
    fresh2.load_state_dict(base_sd, strict=False)
    fresh2.load_adapters(str(tmp_path / "lin.pt"), name="lin")
    assert fresh2.get_enabled_adapters() == ["encoder:lin"] and torch.allclose(fresh2.forward(input_signal=audio, input_signal_length=lens)[0], only_lin, atol=1e-5)
    # whole model with adapters through .nemo
    m.save_to(str(tmp_path / "m.nemo"))
    back = EncDecCTCModelBPE.restore_from(str(tmp_path / "m.nemo")).eval()
    assert back.get_enabled_adapters() == m.get_enabled_adapters()
    assert torch.allclose(back.forward(input_signal=audio, input_signal_length=lens)[0], with_ad, atol=1e-5)
    # stand-alone modules and the stochastic-depth strategy
    x = torch.randn(2, 9, 32)
    for ad in (MultiHeadAttentionAdapter(4, 32), RelPositionMultiHeadAttentionAdapter(4, 32, max_rel=3)):
        assert float(ad(x).abs().max()) == 0.0          # zero-initialised output projection
    assert torch.equal(PositionalEncodingAdapter(32, max_len=16)(x), x)
    host = torch.nn.Linear(1, 1).train()
    st = ResidualAddAdapterStrategy(stochastic_depth=1.0)
    assert torch.equal(st(x, torch.nn.Linear(32, 32), module=host), x)
    with pytest.raises(ValueError, match="not one of"):
        m.add_adapter("vocoder:x", {"in_features": 176, "dim": 4})


def test_transcribe_long_audio_in_chunks_merges_tokens_and_frame_indices():
    from speech_b200.models import EncDecCTCModelBPE
    from speech_b200.models.configs import fastconformer_ctc_config

    torch.manual_seed(0)
    m = EncDecCTCModelBPE(fastconformer_ctc_config("small", vocab_size=32, n_layers=1)).eval()
    g = torch.Generator().manual_seed(0)
    long_audio = (0.1 * torch.randn(16000 * 3 + 500, generator=g)).numpy()
    short = long_audio[:8000]
    chunked = m.transcribe([long_audio, short], batch_size=4, return_hypotheses=True, chunk_duration_seconds=1.0)
    parts = m.transcribe([long_audio[:16000], long_audio[16000:32000], long_audio[32000:]], batch_size=4, return_hypotheses=True)
    assert len(chunked) == 2
    want = [int(t) for p in parts for t in (p.y_sequence.tolist() if torch.is_tensor(p.y_sequence) else p.y_sequence)]
    assert [int(t) for t in chunked[0].y_sequence.tolist()] == want                 # the 500-sample sliver joined the third chunk
    assert chunked[1].text == m.transcribe([short], batch_size=1)[0]
    texts = m.transcribe([long_audio], batch_size=2, chunk_duration_seconds=1.0)
    assert isinstance(texts[0], str)


def test_masked_patch_and_crop_or_pad_augmentations_and_front_end_config_records():
    import torch

    from speech_b200.core.config_schemas import to_dictconfig
    from speech_b200.core.instantiate import instantiate
    from speech_b200.modules import configs as C
    from speech_b200.modules.spec_augment import CropOrPadSpectrogramAugmentation, MaskedPatchAugmentation

    torch.manual_seed(0)
    x = torch.ones(3, 4, 50)
    lens = torch.tensor([50, 33, 20])
    y = MaskedPatchAugmentation(patch_size=5, mask_patches=3)(input_spec=x.clone(), length=lens)
    zero = (y == 0).all(1)
    assert zero.sum(1).tolist() == [15, 15, 15]                                        # the same amount masked in every utterance
    for b in range(3):
        cols = zero[b].nonzero().flatten()
        assert int(cols.max()) < int(lens[b]) // 5 * 5 and all(int(zero[b, s:s + 5].sum()) in (0, 5) for s in range(0, 50, 5))   # whole patches, inside the length
    frac = MaskedPatchAugmentation(patch_size=5, mask_patches=0.3)(input_spec=x.clone(), length=lens)
    assert (frac == 0).all(1).sum(1).tolist() == [10, 10, 10]                          # 30 % of the shortest (20) = 6 frames → 2 patches
    many = MaskedPatchAugmentation(patch_size=5, mask_patches=9)(input_spec=x.clone(), length=lens)
    assert (many == 0).all(1).sum(1).tolist() == [20, 20, 20]                          # capped by the shortest utterance
    fm = MaskedPatchAugmentation(patch_size=5, mask_patches=1, freq_masks=1, freq_width=2)(input_spec=x.clone(), length=lens)
    assert fm.shape == x.shape
    with pytest.raises(ValueError):
        MaskedPatchAugmentation(mask_patches=-1)

    ramp = torch.arange(50.0).expand(2, 3, 50).contiguous()
    crop, cl = CropOrPadSpectrogramAugmentation(20)(input_signal=ramp, length=torch.tensor([50, 40]))
    assert crop.shape == (2, 3, 20) and cl.tolist() == [20, 20] and bool((crop[:, :, 1:] - crop[:, :, :-1] == 1).all())
    pad, pl = CropOrPadSpectrogramAugmentation(55)(input_signal=ramp + 1, length=torch.tensor([50, 40]))
    assert pad.shape == (2, 3, 55) and pl.tolist() == [55, 55] and float(pad[0, 0, :2].sum()) == 0 and float(pad[0, 0, 2]) == 1 and float(pad[0, 0, 52:].sum()) == 0

    pre = instantiate(to_dictconfig(C.AudioToMelSpectrogramPreprocessorConfig(features=32, dither=0.0)))
    feats, fl = pre(input_signal=torch.randn(2, 3200), length=torch.tensor([3200, 1600]))
    assert feats.shape[1] == 32 and fl.tolist() == [20, 10]
    aug = instantiate(to_dictconfig(C.MaskedPatchAugmentationConfig(patch_size=4, mask_patches=2)))
    assert isinstance(aug, MaskedPatchAugmentation) and aug.patch_size == 4
    assert instantiate(to_dictconfig(C.CropOrPadSpectrogramAugmentationConfig(audio_length=16))).audio_length == 16
    mfcc = instantiate(to_dictconfig(C.AudioToMFCCPreprocessorConfig(n_mfcc=13, n_mels=24)))
    assert mfcc(input_signal=torch.randn(1, 3200), length=torch.tensor([3200]))[0].shape[1] == 13
    sa = instantiate(to_dictconfig(C.SpectrogramAugmentationConfig(freq_masks=1, freq_width=3)))
    assert sa(input_spec=torch.ones(1, 8, 10), length=torch.tensor([10])).shape == (1, 8, 10)
