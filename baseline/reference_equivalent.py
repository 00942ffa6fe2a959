"""Reference-equivalent FastConformer-TDT trainer built only from library ops (eager PyTorch + cuBLAS / cuDNN + NCCL).

The reference framework cannot be installed offline (its Lightning / Hydra / OmegaConf / Lhotse dependencies are missing), so
its headline training step is restated here from the same library calls it makes, module by module:

* features: ``torch.stft`` + mel filterbank + log + per-feature normalisation
  (``nemo/collections/asr/parts/preprocessing/features.py``, ``FilterbankFeatures.forward``);
* sub-sampling: ``nn.Conv2d`` depthwise-striding stack + ``nn.Linear`` (``parts/submodules/subsampling.py:184-257``);
* Conformer layer: ``nn.LayerNorm`` / ``nn.Linear`` feed-forward halves, relative-position attention as two ``torch.matmul``
  + ``rel_shift`` + softmax (the default, non-SDPA branch of ``parts/submodules/multi_head_attention.py:279-361``; set
  ``REFEQ_SDPA=1`` for its ``scaled_dot_product_attention`` branch), ``nn.Conv1d`` + GLU + depthwise ``nn.Conv1d`` +
  ``nn.BatchNorm1d`` (``SyncBatchNorm`` under DDP) + SiLU (``parts/submodules/conformer_modules.py``);
* prediction network: ``nn.Embedding`` + 2-layer ``nn.LSTM`` (cuDNN) (``modules/rnnt.py``), joint: two ``nn.Linear`` + ReLU +
  ``nn.Linear`` over the full ``[B, T, U+1, V]`` lattice, in sub-batches of ``fused_batch_size`` utterances as the
  reference recipe does (``examples/asr/conf/fastconformer/fast-conformer_transducer_bpe.yaml``);
* loss: the reference's OWN Numba TDT kernels (``parts/numba/rnnt_loss/rnnt_pytorch.py:TDTLossNumba``), loaded unmodified from
  the reference tree when it is present (that sub-package only needs numba and torch), otherwise a PyTorch wavefront;
* ``torch.optim.AdamW`` + Noam schedule, ``clip_grad_norm_``, bf16 autocast with fp32 parameters,
  ``DistributedDataParallel`` (25 MB buckets) over NCCL.

Results obtained with this file are labelled "reference-equivalent (eager PyTorch + NCCL)", never "reference".
"""
from __future__ import annotations

import importlib
import math
import os
import sys
import types
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


# ----------------------------------------------------------------------------------------------------------- features
class MelFeatures(nn.Module):
    def __init__(self, sr=16000, n_fft=512, win=400, hop=160, n_mels=80, preemph=0.97, dither=1e-5):
        super().__init__()
        self.n_fft, self.win, self.hop, self.preemph, self.dither = n_fft, win, hop, preemph, dither
        self.register_buffer("window", torch.hann_window(win, periodic=False), persistent=False)
        self.register_buffer("fb", self._mel_fb(sr, n_fft, n_mels), persistent=False)

    @staticmethod
    def _mel_fb(sr, n_fft, n_mels):
        # Slaney-style triangular filters with area normalisation (what librosa.filters.mel produces)
        def hz2mel(f):
            f = torch.as_tensor(f, dtype=torch.float64)
            lin = f / (200.0 / 3)
            log = 15.0 + torch.log(f.clamp(min=1e-10) / 1000.0) / (math.log(6.4) / 27.0)
            return torch.where(f >= 1000.0, log, lin)

        def mel2hz(m):
            lin = m * (200.0 / 3)
            log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
            return torch.where(m >= 15.0, log, lin)

        freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
        mels = torch.linspace(float(hz2mel(0.0)), float(hz2mel(sr / 2)), n_mels + 2, dtype=torch.float64)
        hz = mel2hz(mels)
        fb = torch.zeros(n_mels, n_fft // 2 + 1, dtype=torch.float64)
        for i in range(n_mels):
            lo, ce, hi = hz[i], hz[i + 1], hz[i + 2]
            up = (freqs - lo) / (ce - lo)
            down = (hi - freqs) / (hi - ce)
            fb[i] = torch.clamp(torch.minimum(up, down), min=0.0) * (2.0 / (hi - lo))
        return fb.float()

    @torch.no_grad()
    def forward(self, x: torch.Tensor, lens: torch.Tensor):
        with torch.autocast("cuda", enabled=False):
            x = x.float()
            if self.training and self.dither > 0:
                x = x + self.dither * torch.randn_like(x)
            x = torch.cat([x[:, :1], x[:, 1:] - self.preemph * x[:, :-1]], dim=1)
            t = torch.arange(x.shape[1], device=x.device)[None, :] < lens[:, None]
            x = x * t
            win = F.pad(self.window, ((self.n_fft - self.win) // 2, (self.n_fft - self.win + 1) // 2))
            spec = torch.stft(x, self.n_fft, hop_length=self.hop, win_length=self.n_fft, window=win, center=True,
                              return_complex=True)
            power = spec.real.pow(2) + spec.imag.pow(2)
            mel = torch.log(torch.matmul(self.fb, power) + 2.0 ** -24)
            flen = lens // self.hop + 1
            m = (torch.arange(mel.shape[2], device=x.device)[None, :] < flen[:, None]).unsqueeze(1)
            cnt = flen.clamp(min=1)[:, None, None].float()
            mean = (mel * m).sum(2, keepdim=True) / cnt
            var = ((mel - mean).pow(2) * m).sum(2, keepdim=True) / (cnt - 1).clamp(min=1)
            mel = ((mel - mean) / (var.sqrt() + 1e-5)) * m
            return mel, flen


class SpecAugment(nn.Module):
    def __init__(self, freq_masks=2, freq_width=27, time_masks=10, time_width=0.05):
        super().__init__()
        self.fm, self.fw, self.tm, self.tw = freq_masks, freq_width, time_masks, time_width

    @torch.no_grad()
    def forward(self, x, lens):
        B, Fq, T = x.shape
        dev = x.device
        f0 = torch.randint(0, Fq - self.fw, (B, self.fm), device=dev)
        fw = torch.randint(0, self.fw + 1, (B, self.fm), device=dev)
        fi = torch.arange(Fq, device=dev)[None, None, :]
        fmask = ((fi >= f0[..., None]) & (fi < (f0 + fw)[..., None])).any(1)
        tw_max = (lens.float() * self.tw).long().clamp(min=1)
        t0 = (torch.rand(B, self.tm, device=dev) * (lens[:, None] - tw_max[:, None]).clamp(min=1)).long()
        tw = (torch.rand(B, self.tm, device=dev) * (tw_max[:, None] + 1)).long()
        ti = torch.arange(T, device=dev)[None, None, :]
        tmask = ((ti >= t0[..., None]) & (ti < (t0 + tw)[..., None])).any(1)
        return x.masked_fill(fmask[:, :, None] | tmask[:, None, :], 0.0)


# ----------------------------------------------------------------------------------------------------------- encoder
class DwStridingSubsampling(nn.Module):
    def __init__(self, feat_in=80, d_model=1024, channels=256):
        super().__init__()
        layers = [nn.Conv2d(1, channels, 3, 2, 1), nn.ReLU(True)]
        for _ in range(2):
            layers += [nn.Conv2d(channels, channels, 3, 2, 1, groups=channels), nn.Conv2d(channels, channels, 1), nn.ReLU(True)]
        self.conv = nn.Sequential(*layers)
        self.out = nn.Linear(channels * (feat_in // 8), d_model)

    def forward(self, x, lens):           # x [B, T, F]
        for _ in range(3):
            lens = (lens + 2 * 1 - 3) // 2 + 1
        x = self.conv(x.unsqueeze(1))
        b, c, t, f = x.shape
        return self.out(x.transpose(1, 2).reshape(b, t, c * f)), lens


class RelPosEncoding(nn.Module):
    def __init__(self, d_model, dropout):
        super().__init__()
        self.d_model, self.drop = d_model, nn.Dropout(dropout)

    def forward(self, x):
        T = x.shape[1]
        pos = torch.arange(T - 1, -T, -1, dtype=torch.float32, device=x.device).unsqueeze(1)
        div = torch.exp(torch.arange(0, self.d_model, 2, dtype=torch.float32, device=x.device) * -(math.log(10000.0) / self.d_model))
        pe = torch.zeros(2 * T - 1, self.d_model, device=x.device)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        return self.drop(x), self.drop(pe.unsqueeze(0).to(x.dtype))


class RelPosMHA(nn.Module):
    def __init__(self, d_model, heads, dropout):
        super().__init__()
        self.h, self.dk = heads, d_model // heads
        self.linear_q, self.linear_k, self.linear_v = nn.Linear(d_model, d_model), nn.Linear(d_model, d_model), nn.Linear(d_model, d_model)
        self.linear_out = nn.Linear(d_model, d_model)
        self.linear_pos = nn.Linear(d_model, d_model, bias=False)
        self.pos_bias_u = nn.Parameter(torch.zeros(heads, self.dk))
        self.pos_bias_v = nn.Parameter(torch.zeros(heads, self.dk))
        self.drop = nn.Dropout(dropout)
        self.p = dropout
        self.sdpa = os.environ.get("REFEQ_SDPA", "0") == "1"

    @staticmethod
    def rel_shift(x):
        b, h, qlen, pos_len = x.size()
        x = F.pad(x, pad=(1, 0))
        x = x.view(b, h, -1, qlen)[:, :, 1:].view(b, h, qlen, pos_len)
        return x

    def forward(self, x, pos_emb, mask):   # mask [B, T, T] True = masked
        B, T, _ = x.shape
        q = self.linear_q(x).view(B, T, self.h, self.dk)
        k = self.linear_k(x).view(B, T, self.h, self.dk).transpose(1, 2)
        v = self.linear_v(x).view(B, T, self.h, self.dk).transpose(1, 2)
        p = self.linear_pos(pos_emb).view(pos_emb.shape[0], -1, self.h, self.dk).transpose(1, 2)
        q_u = (q + self.pos_bias_u).transpose(1, 2)
        q_v = (q + self.pos_bias_v).transpose(1, 2)
        matrix_bd = self.rel_shift(torch.matmul(q_v, p.transpose(-2, -1)))
        scale = 1.0 / math.sqrt(self.dk)
        if self.sdpa:
            bd = matrix_bd[:, :, :, :T] * scale
            bd = bd.masked_fill(mask.unsqueeze(1), float("-inf"))
            out = F.scaled_dot_product_attention(q_u, k, v, attn_mask=bd, dropout_p=self.p if self.training else 0.0)
            all_masked = mask.all(-1)
            out = out.masked_fill(all_masked[:, None, :, None], 0.0)
        else:
            matrix_ac = torch.matmul(q_u, k.transpose(-2, -1))
            scores = (matrix_ac + matrix_bd[:, :, :, :T]) * scale
            scores = scores.masked_fill(mask.unsqueeze(1), -10000.0)
            attn = torch.softmax(scores, dim=-1).masked_fill(mask.unsqueeze(1), 0.0)
            out = torch.matmul(self.drop(attn), v)
        return self.linear_out(out.transpose(1, 2).reshape(B, T, self.h * self.dk))


class FeedForward(nn.Module):
    def __init__(self, d_model, d_ff, dropout):
        super().__init__()
        self.linear1, self.linear2, self.drop = nn.Linear(d_model, d_ff), nn.Linear(d_ff, d_model), nn.Dropout(dropout)

    def forward(self, x):
        return self.linear2(self.drop(F.silu(self.linear1(x))))


class ConvModule(nn.Module):
    def __init__(self, d_model, k):
        super().__init__()
        self.pointwise_conv1 = nn.Conv1d(d_model, 2 * d_model, 1)
        self.depthwise_conv = nn.Conv1d(d_model, d_model, k, padding=(k - 1) // 2, groups=d_model)
        self.batch_norm = nn.BatchNorm1d(d_model)
        self.pointwise_conv2 = nn.Conv1d(d_model, d_model, 1)

    def forward(self, x, pad_mask):
        x = x.transpose(1, 2)
        x = F.glu(self.pointwise_conv1(x), dim=1)
        x = x.masked_fill(pad_mask.unsqueeze(1), 0.0)
        x = F.silu(self.batch_norm(self.depthwise_conv(x)))
        return self.pointwise_conv2(x).transpose(1, 2)


class ConformerLayer(nn.Module):
    def __init__(self, d_model, d_ff, heads, k, dropout):
        super().__init__()
        self.norm_feed_forward1, self.feed_forward1 = nn.LayerNorm(d_model), FeedForward(d_model, d_ff, dropout)
        self.norm_self_att, self.self_attn = nn.LayerNorm(d_model), RelPosMHA(d_model, heads, dropout)
        self.norm_conv, self.conv = nn.LayerNorm(d_model), ConvModule(d_model, k)
        self.norm_feed_forward2, self.feed_forward2 = nn.LayerNorm(d_model), FeedForward(d_model, d_ff, dropout)
        self.norm_out, self.drop = nn.LayerNorm(d_model), nn.Dropout(dropout)

    def forward(self, x, pos_emb, att_mask, pad_mask):
        x = x + 0.5 * self.drop(self.feed_forward1(self.norm_feed_forward1(x)))
        x = x + self.drop(self.self_attn(self.norm_self_att(x), pos_emb, att_mask))
        x = x + self.drop(self.conv(self.norm_conv(x), pad_mask))
        x = x + 0.5 * self.drop(self.feed_forward2(self.norm_feed_forward2(x)))
        return self.norm_out(x)


class ConformerEncoder(nn.Module):
    def __init__(self, n_layers=24, d_model=1024, heads=8, d_ff=4096, k=9, dropout=0.1, feat_in=80):
        super().__init__()
        self.pre_encode = DwStridingSubsampling(feat_in, d_model)
        self.pos_enc = RelPosEncoding(d_model, dropout)
        self.layers = nn.ModuleList(ConformerLayer(d_model, d_ff, heads, k, dropout) for _ in range(n_layers))

    def forward(self, feats, flen):
        x, lens = self.pre_encode(feats.transpose(1, 2), flen)
        T = x.shape[1]
        x, pos_emb = self.pos_enc(x)
        pad = torch.arange(T, device=x.device)[None, :] >= lens[:, None]
        att = pad.unsqueeze(1) | pad.unsqueeze(2)
        for layer in self.layers:
            x = layer(x, pos_emb, att, pad)
        return x, lens


# ----------------------------------------------------------------------------------------------------------- transducer
class PredictionNet(nn.Module):
    def __init__(self, vocab, hidden=640, layers=2, dropout=0.0):
        super().__init__()
        self.embed = nn.Embedding(vocab + 1, hidden, padding_idx=vocab)
        self.lstm = nn.LSTM(hidden, hidden, num_layers=layers, dropout=dropout, batch_first=False)
        self.drop = nn.Dropout(dropout)

    def forward(self, targets):           # [B, U] -> [B, U+1, H]
        y = self.embed(targets)
        y = torch.cat([torch.zeros_like(y[:, :1]), y], dim=1)
        g, _ = self.lstm(y.transpose(0, 1))
        return self.drop(g).transpose(0, 1)


class Joint(nn.Module):
    def __init__(self, enc=1024, pred=640, hidden=640, n_out=1030, dropout=0.0):
        super().__init__()
        self.enc, self.pred = nn.Linear(enc, hidden), nn.Linear(pred, hidden)
        self.joint_net = nn.Sequential(nn.ReLU(True), nn.Dropout(dropout), nn.Linear(hidden, n_out))

    def forward(self, f, g):              # f [b, T, hidden] (projected), g [b, U1, hidden] (projected)
        return self.joint_net(f.unsqueeze(2) + g.unsqueeze(1))


def load_reference_tdt_loss(ref_root: str):
    """``TDTLossNumba`` of the reference tree, imported without running the reference's top-level packages (which need
    Lightning / Hydra): parent packages are registered as empty modules whose ``__path__`` points at the real directories."""
    base = os.path.join(ref_root, "nemo")
    if not os.path.isdir(os.path.join(base, "collections", "asr", "parts", "numba", "rnnt_loss")):
        return None
    chain = ["nemo", "nemo.collections", "nemo.collections.asr", "nemo.collections.asr.parts"]
    for name in chain:
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = [os.path.join(ref_root, *name.split("."))]
            sys.modules[name] = m
    try:
        mod = importlib.import_module("nemo.collections.asr.parts.numba.rnnt_loss.rnnt_pytorch")
        return mod.TDTLossNumba
    except Exception:  # noqa: BLE001
        for name in chain:
            sys.modules.pop(name, None)
        return None


def tdt_loss_wavefront(logits, targets, f_len, y_len, blank, durations: Sequence[int], sigma: float):
    """TDT negative log-likelihood per utterance: forward recursion over anti-diagonals t + u = n, vectorised over the batch
    and the diagonal; autograd supplies the gradient.  Fallback when the reference's Numba kernels cannot be loaded."""
    B, T, U1, _ = logits.shape
    D = len(durations)
    dev = logits.device
    lp = torch.log_softmax(logits[..., :-D].float(), dim=-1) - sigma
    dp = torch.log_softmax(logits[..., -D:].float(), dim=-1)
    blank_lp = lp[..., blank]
    tgt = torch.cat([targets, targets.new_zeros(B, 1)], dim=1)[:, :U1].long()
    label_lp = lp.gather(-1, tgt[:, None, :, None].expand(B, T, U1, 1)).squeeze(-1)
    NEG = -1e30
    alpha = torch.full((B, T + 1, U1), NEG, device=dev)
    alpha[:, 0, 0] = 0.0
    fl = f_len.long().to(dev)
    for n in range(1, T + U1):
        t = torch.arange(max(0, n - U1 + 1), min(n, T) + 1, device=dev)
        u = n - t
        terms = []
        for di, d in enumerate(durations):
            tp = t - d
            ok = (tp >= 0) & (tp < T)
            tpc = tp.clamp(0, T - 1)
            okb = ok[None, :] & (tp[None, :] < fl[:, None])      # the source frame lies inside the utterance
            if d > 0:      # blank keeps u and advances d frames (the only way into the terminal row t = f_len)
                v = alpha[:, tpc, u] + blank_lp[:, tpc, u] + dp[:, tpc, u, di]
                terms.append(torch.where(okb & (t[None, :] <= fl[:, None]), v, torch.full_like(v, NEG)))
            okl = okb & (u > 0)[None, :] & (t[None, :] < fl[:, None])
            uc = (u - 1).clamp(min=0)
            v = alpha[:, tpc, uc] + label_lp[:, tpc, uc] + dp[:, tpc, uc, di]
            terms.append(torch.where(okl, v, torch.full_like(v, NEG)))
        new = torch.logsumexp(torch.stack(terms, 0), 0)
        alpha = alpha.clone()
        alpha[:, t, u] = new
    bi = torch.arange(B, device=dev)
    return -alpha[bi, f_len.long().clamp(max=T), y_len.long().clamp(max=U1 - 1)]


class RefEqTDT(nn.Module):
    def __init__(self, vocab=1024, n_layers=24, d_model=1024, heads=8, d_ff=4096, k=9, dropout=0.1, pred_dropout=0.0,
                 joint_dropout=0.0, durations=(0, 1, 2, 3, 4), sigma=0.02, fused_batch_size=4, ref_root: Optional[str] = None):
        super().__init__()
        self.vocab, self.durations, self.sigma, self.fused = vocab, list(durations), sigma, fused_batch_size
        self.features, self.spec_aug = MelFeatures(), SpecAugment()
        self.encoder = ConformerEncoder(n_layers, d_model, heads, d_ff, k, dropout)
        self.decoder = PredictionNet(vocab, 640, 2, pred_dropout)
        self.joint = Joint(d_model, 640, 640, vocab + 1 + len(durations), joint_dropout)
        cls = load_reference_tdt_loss(ref_root) if ref_root else None
        self.loss_kind = "reference Numba TDT kernels" if cls is not None else "PyTorch wavefront"
        self.loss_fn = cls(blank=vocab, durations=list(durations), reduction="none", sigma=sigma) if cls is not None else None

    def forward(self, audio, alen, tokens, tlen):
        feats, flen = self.features(audio, alen)
        if self.training:
            feats = self.spec_aug(feats, flen)
        enc, elen = self.encoder(feats, flen)
        pred = self.decoder(tokens)
        f, g = self.joint.enc(enc), self.joint.pred(pred)
        B = f.shape[0]
        total = f.new_zeros((), dtype=torch.float32)
        for s in range(0, B, self.fused):
            sl = slice(s, min(B, s + self.fused))
            tmax, umax = int(elen[sl].max()), int(tlen[sl].max())
            logits = self.joint(f[sl, :tmax], g[sl, :umax + 1]).float()
            if self.loss_fn is not None:
                l = self.loss_fn(logits, tokens[sl, :umax].long().contiguous(), elen[sl].long(), tlen[sl].long())
            else:
                l = tdt_loss_wavefront(logits, tokens[sl, :umax], elen[sl], tlen[sl], self.vocab, self.durations, self.sigma)
            total = total + l.sum()
        return total / B


def build(device, world: int, local_rank: int, n_layers: Optional[int], dropout: float, ref_root: str, lr: float = 5.0,
          warmup_steps: int = 10000, d_model: int = 1024):
    """Model (DDP-wrapped when world > 1), optimizer, scheduler and one ``step(batch) -> loss`` callable."""
    model = RefEqTDT(n_layers=n_layers or 24, dropout=dropout, ref_root=ref_root).to(device)
    net = model
    if world > 1:
        model = nn.SyncBatchNorm.convert_sync_batchnorm(model)
        net = nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=25, gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.98), weight_decay=1e-3)
    noam = lambda s: (d_model ** -0.5) * min(max(s, 1) ** -0.5, max(s, 1) * warmup_steps ** -1.5)  # noqa: E731
    sched = torch.optim.lr_scheduler.LambdaLR(opt, noam)

    def step(batch):
        audio, alen, tokens, tlen = batch
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(audio, alen, tokens, tlen)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()

    return model, step


# ----------------------------------------------------------------------------------------------------------- speech-LLM
class RefEqSALM(nn.Module):
    """Speech-LLM the way the reference assembles it from libraries: mel features -> Conformer encoder (above) -> linear
    projection to the LLM width; text embedded by the LLM's table; audio embeddings spliced over the placeholder token of every
    row (left padded); Hugging Face ``Qwen3ForCausalLM`` on ``inputs_embeds`` with ``labels`` (logits and cross entropy at every
    position, as ``transformers`` computes them)."""

    def __init__(self, llm_cfg: dict, enc_layers: int = 32, d_model: int = 1024, n_mels: int = 128, dropout: float = 0.1,
                 placeholder_id: int = 0, pad_id: int = 0):
        super().__init__()
        from transformers import Qwen3Config, Qwen3ForCausalLM

        self.features = MelFeatures(n_mels=n_mels)
        self.encoder = ConformerEncoder(enc_layers, d_model, 8, 4 * d_model, 9, dropout, feat_in=n_mels)
        cfg = Qwen3Config(**{k: v for k, v in llm_cfg.items() if k not in ("qk_norm", "model_type")})
        self.llm = Qwen3ForCausalLM(cfg)
        self.proj = nn.Linear(d_model, cfg.hidden_size)
        self.placeholder_id, self.pad_id = placeholder_id, pad_id

    def forward(self, audios, audio_lens, input_ids, loss_mask):
        feats, flen = self.features(audios, audio_lens)
        enc, elen = self.encoder(feats, flen)
        aud = self.proj(enc)
        emb_table = self.llm.get_input_embeddings()
        rows, tgts = [], []
        a = 0
        elen_l = elen.tolist()
        for b in range(input_ids.shape[0]):
            ids = input_ids[b]
            keep = ids != self.pad_id
            ids, lm = ids[keep], loss_mask[b][keep]
            pos = (ids == self.placeholder_id).nonzero().flatten().tolist()
            text = emb_table(ids)
            tgt = torch.where(lm.bool(), ids, torch.full_like(ids, -100))
            parts, tparts, prev = [], [], 0
            for p in pos:
                n = int(elen_l[a])
                parts += [text[prev:p], aud[a, :n].to(text.dtype)]
                tparts += [tgt[prev:p], torch.full((n,), -100, dtype=tgt.dtype, device=tgt.device)]
                prev, a = p + 1, a + 1
            parts.append(text[prev:])
            tparts.append(tgt[prev:])
            rows.append(torch.cat(parts))
            tgts.append(torch.cat(tparts))
        L = max(r.shape[0] for r in rows)
        H = rows[0].shape[1]
        emb = rows[0].new_zeros((len(rows), L, H))
        labels = torch.full((len(rows), L), -100, dtype=torch.long, device=emb.device)
        mask = torch.zeros((len(rows), L), dtype=torch.long, device=emb.device)
        for b, (r, t) in enumerate(zip(rows, tgts)):
            emb[b, L - r.shape[0]:] = r
            labels[b, L - r.shape[0]:] = t
            mask[b, L - r.shape[0]:] = 1
        out = self.llm(inputs_embeds=emb, attention_mask=mask, labels=labels)
        return out.loss, emb.shape[0] * emb.shape[1]
