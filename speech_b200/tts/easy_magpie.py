"""Decoder-only text-to-speech on a language-model backbone, with a hybrid state-space / attention decoder.

* ``Mamba2Block`` — selective state-space layer in its "state-space dual" form.  Per head ``h`` with a state ``S [P, N]``:
  ``S_t = exp(dt_t A_h) S_{t-1} + dt_t x_t B_t^T``, ``y_t = S_t C_t + D_h x_t``; ``x, B, C`` pass a causal depthwise convolution
  and SiLU first, the output is gated by ``SiLU(z)``, RMS-normalised and projected.  Training evaluates the recurrence chunk by
  chunk: inside a chunk as a masked, decay-weighted ``(C B^T)`` product (GEMM-shaped work), between chunks through the carried
  state; ``step`` is the O(1) recurrence for decoding with a (convolution window, state) cache.  Both give the same numbers.
* ``NemotronHDecoder`` — a stack described by a pattern string: ``M`` = Mamba-2 block, ``*`` = causal self-attention (rotary,
  grouped KV heads), ``-`` = gated MLP, ``E`` = mixture-of-experts block (``NemotronHMoE``); every block is pre-normalised with a residual connection.
* ``EasyMagpieTTSModel`` — one sequence ``[text tokens | audio frames]``: text tokens use the text embedding table, an audio
  frame is the sum of its per-codebook embeddings; the backbone is a ``CausalLM`` transformer or the hybrid decoder; one linear
  head per codebook predicts the next frame.  Training: cross-entropy on the audio positions; inference: autoregressive sampling
  with the backbone's caches until the first codebook emits EOS.

Reference: ``tts/models/easy_magpietts.py`` (sequence layout, per-codebook heads, sampling loop),
``tts/modules/nemotron_h_decoder.py`` (hybrid pattern, Mamba-2 mixer; the optional mamba-ssm / causal-conv1d CUDA packages
``:38-89`` are not needed here: the chunked form maps to batched GEMMs).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import DictConfig, cfg_get
from ..core.modelpt import ModelPT
from ..speechlm.llm import Attention, CausalLM, LLMConfig, MLP, RMSNorm, rope_tables


class Mamba2Block(nn.Module):
    def __init__(self, d_model: int, d_state: int = 16, d_conv: int = 4, expand: int = 2, head_dim: int = 16, n_groups: int = 1,
                 chunk_size: int = 64):
        super().__init__()
        self.d_inner = expand * d_model
        if self.d_inner % head_dim:
            raise ValueError("expand * d_model must be a multiple of head_dim")
        self.H, self.P, self.N, self.G, self.k, self.chunk = self.d_inner // head_dim, head_dim, d_state, n_groups, d_conv, chunk_size
        self.conv_dim = self.d_inner + 2 * self.G * self.N
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner + 2 * self.G * self.N + self.H, bias=False)
        self.conv_w = nn.Parameter(torch.randn(self.conv_dim, d_conv) * d_conv ** -0.5)
        self.conv_b = nn.Parameter(torch.zeros(self.conv_dim))
        self.A_log = nn.Parameter(torch.log(torch.linspace(1.0, 16.0, self.H)))
        self.D = nn.Parameter(torch.ones(self.H))
        dt = torch.exp(torch.rand(self.H) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))                     # inverse softplus
        self.norm = RMSNorm(self.d_inner)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False)

    def _split(self, u):
        z, xbc, dt = torch.split(self.in_proj(u), [self.d_inner, self.conv_dim, self.H], dim=-1)
        return z, xbc, F.softplus(dt.float() + self.dt_bias.float())

    def _heads(self, xbc):
        x, B, C = torch.split(xbc, [self.d_inner, self.G * self.N, self.G * self.N], dim=-1)
        sh = x.shape[:-1]
        x = x.reshape(*sh, self.H, self.P).float()
        rep = self.H // self.G
        B = B.reshape(*sh, self.G, self.N).float().repeat_interleave(rep, dim=-2)
        C = C.reshape(*sh, self.G, self.N).float().repeat_interleave(rep, dim=-2)
        return x, B, C

    def forward(self, u: torch.Tensor, cache: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
        """u [B, T, d].  With a ``cache`` dict the call continues from (and updates) its convolution window and state."""
        if cache is not None and u.shape[1] == 1 and "ssm" in cache:
            return self.step(u, cache)
        Bsz, T, _ = u.shape
        z, xbc, dt = self._split(u)
        prev = cache.get("conv") if cache else None
        pad = prev if prev is not None else xbc.new_zeros(Bsz, self.k - 1, self.conv_dim)
        seq = torch.cat([pad, xbc], dim=1)
        conv = F.conv1d(seq.transpose(1, 2), self.conv_w.unsqueeze(1).to(seq.dtype), self.conv_b.to(seq.dtype), groups=self.conv_dim)
        x, Bm, Cm = self._heads(F.silu(conv.transpose(1, 2)))
        la = -torch.exp(self.A_log.float()) * dt                                            # log decay per step  [B, T, H]
        S = cache["ssm"].float() if cache and "ssm" in cache else x.new_zeros(Bsz, self.H, self.P, self.N)
        ys = []
        for s in range(0, T, self.chunk):
            e = min(T, s + self.chunk)
            xc, Bc, Cc, dtc = x[:, s:e], Bm[:, s:e], Cm[:, s:e], dt[:, s:e]
            L = la[:, s:e].cumsum(1)                                                        # [B, c, H] log decay from chunk start
            # inside the chunk: y_t += sum_{r<=t} (C_t . B_r) exp(L_t - L_r) dt_r x_r
            w = torch.einsum("bthn,brhn->bhtr", Cc, Bc)
            dec = L.permute(0, 2, 1).unsqueeze(-1) - L.permute(0, 2, 1).unsqueeze(-2)       # [B, H, t, r]
            causal = torch.ones(e - s, e - s, dtype=torch.bool, device=u.device).tril()
            w = w * torch.exp(dec.masked_fill(~causal, float("-inf"))) * dtc.permute(0, 2, 1).unsqueeze(-2)
            y = torch.einsum("bhtr,brhp->bthp", w, xc)
            # carried state: y_t += exp(L_t) C_t S ;  S' = exp(L_end) S + sum_r exp(L_end - L_r) dt_r x_r B_r^T
            y = y + torch.einsum("bthn,bhpn->bthp", Cc * torch.exp(L).unsqueeze(-1), S)
            tail = torch.exp(L[:, -1:] - L) * dtc                                           # [B, c, H]
            S = torch.exp(L[:, -1]).unsqueeze(-1).unsqueeze(-1) * S + torch.einsum("brhp,brhn->bhpn", xc * tail.unsqueeze(-1), Bc)
            ys.append(y + self.D.float().view(1, 1, -1, 1) * xc)
        y = torch.cat(ys, dim=1).reshape(Bsz, T, self.d_inner).to(u.dtype)
        if cache is not None:
            cache["conv"], cache["ssm"] = seq[:, -(self.k - 1):].detach(), S.detach()
        return self.out_proj(self.norm(y * F.silu(z)))

    def step(self, u: torch.Tensor, cache: Dict[str, torch.Tensor]) -> torch.Tensor:
        z, xbc, dt = self._split(u)                                                         # [B, 1, .]
        win = torch.cat([cache["conv"], xbc], dim=1)                                        # [B, k, C]
        conv = (win * self.conv_w.t().to(win.dtype)).sum(1) + self.conv_b.to(win.dtype)
        x, Bm, Cm = self._heads(F.silu(conv))                                               # [B, H, P] / [B, H, N]
        dt1 = dt[:, 0]
        a = torch.exp(-torch.exp(self.A_log.float()) * dt1)
        S = a.unsqueeze(-1).unsqueeze(-1) * cache["ssm"].float() + torch.einsum("bhp,bhn->bhpn", x * dt1.unsqueeze(-1), Bm)
        y = torch.einsum("bhpn,bhn->bhp", S, Cm) + self.D.float().view(1, -1, 1) * x
        cache["conv"], cache["ssm"] = win[:, 1:], S
        y = y.reshape(u.shape[0], 1, self.d_inner).to(u.dtype)
        return self.out_proj(self.norm(y * F.silu(z)))


class NemotronHMoE(nn.Module):
    """Mixture-of-experts feed-forward block of the hybrid decoder (pattern letter ``E``).  The router scores every expert with a
    sigmoid; experts are arranged in ``n_group`` groups, a group's score is the sum of its two best (bias-corrected) experts, only
    the ``topk_group`` best groups stay eligible and the ``top_k`` best eligible experts are chosen.  The mixing weights are the
    uncorrected sigmoid scores of the chosen experts, optionally normalised to sum to one, times ``routed_scaling_factor``.  Experts
    are plain two-layer MLPs (``down(act(up(x)))``) kept as stacked weights so that the tokens of one expert, after a sort by
    expert, are one GEMM; a shared expert sees every token.
    Reference: ``tts/modules/nemotron_h_decoder.py`` (``NemotronHTopkRouter``, ``NemotronHMOE``)."""

    def __init__(self, hidden_size: int, n_routed_experts: int = 8, num_experts_per_tok: int = 2, moe_intermediate_size: int = 1024,
                 moe_shared_expert_intermediate_size: int = 2048, n_group: int = 1, topk_group: int = 1, routed_scaling_factor: float = 1.0,
                 norm_topk_prob: bool = True, mlp_hidden_act: str = "silu", initializer_range: float = 0.02):
        super().__init__()
        if n_routed_experts % n_group:
            raise ValueError(f"{n_routed_experts} experts do not split into {n_group} groups")
        self.E, self.k, self.n_group, self.topk_group = n_routed_experts, num_experts_per_tok, n_group, topk_group
        self.scale, self.norm_topk_prob = routed_scaling_factor, norm_topk_prob
        self.act = {"silu": F.silu, "gelu": F.gelu, "relu": F.relu, "relu2": lambda v: F.relu(v).square()}[mlp_hidden_act]
        self.router = nn.Parameter(torch.empty(n_routed_experts, hidden_size).normal_(std=initializer_range))
        self.register_buffer("e_score_correction_bias", torch.zeros(n_routed_experts))
        self.up = nn.Parameter(torch.empty(n_routed_experts, moe_intermediate_size, hidden_size).normal_(std=initializer_range))
        self.down = nn.Parameter(torch.empty(n_routed_experts, hidden_size, moe_intermediate_size).normal_(std=initializer_range))
        self.shared_up = nn.Linear(hidden_size, moe_shared_expert_intermediate_size, bias=False)
        self.shared_down = nn.Linear(moe_shared_expert_intermediate_size, hidden_size, bias=False)

    def route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """x [N, H] → (expert indices [N, k], mixing weights [N, k])."""
        scores = F.linear(x.float(), self.router.float()).sigmoid()
        with torch.no_grad():
            choice = scores + self.e_score_correction_bias
            if self.n_group > 1:
                per = self.E // self.n_group
                g = choice.view(-1, self.n_group, per).topk(min(2, per), dim=-1)[0].sum(-1)
                keep = torch.zeros_like(g).scatter_(1, g.topk(self.topk_group, dim=-1)[1], 1.0)
                choice = choice.masked_fill(keep.unsqueeze(-1).expand(-1, -1, per).reshape(-1, self.E) == 0, 0.0)
            idx = choice.topk(self.k, dim=-1)[1]
        w = scores.gather(1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return idx, w * self.scale

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        h = x.reshape(-1, shape[-1])
        idx, w = self.route(h)
        flat = idx.reshape(-1)
        order = flat.argsort(stable=True)
        token = order // self.k
        counts = torch.bincount(flat, minlength=self.E).tolist()
        rows = h[token]
        out = torch.zeros_like(h, dtype=torch.float32)
        o = 0
        for e, n in enumerate(counts):
            if n:
                y = F.linear(self.act(F.linear(rows[o:o + n], self.up[e].to(h.dtype))), self.down[e].to(h.dtype))
                out.index_add_(0, token[o:o + n], y.float() * w.reshape(-1)[order[o:o + n]].unsqueeze(-1))
                o += n
        out = out.to(h.dtype) + self.shared_down(self.act(self.shared_up(h)))
        return out.view(shape)


class _HybridLayer(nn.Module):
    def __init__(self, kind: str, cfg: LLMConfig, mamba: Dict[str, Any], moe: Optional[Dict[str, Any]] = None):
        super().__init__()
        self.kind = kind
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        if kind == "M":
            self.mixer = Mamba2Block(cfg.hidden_size, **mamba)
        elif kind == "*":
            self.mixer = Attention(cfg)
        elif kind == "-":
            self.mixer = MLP(cfg)
        elif kind == "E":
            self.mixer = NemotronHMoE(cfg.hidden_size, **dict(moe or {}))
        else:
            raise ValueError(f"unknown block '{kind}' in the hybrid pattern (use M, *, - and E)")

    def forward(self, x, cos, sin, mask, cache):
        h = self.norm(x)
        if self.kind == "M":
            return x + self.mixer(h, cache)
        if self.kind == "*":
            return x + self.mixer(h, cos, sin, mask, cache)
        return x + self.mixer(h)


class NemotronHDecoder(nn.Module):
    """``forward(inputs_embeds, cache)`` -> hidden states; ``cache`` is a list with one dict per block."""

    def __init__(self, cfg: Any, pattern: str = "M-M*-", mamba: Optional[Dict[str, Any]] = None, moe: Optional[Dict[str, Any]] = None,
                 num_layers: Optional[int] = None):
        super().__init__()
        self.config = cfg if isinstance(cfg, LLMConfig) else LLMConfig(**dict(cfg))
        if num_layers is not None and len(pattern) != num_layers:       # the pattern repeats (or is cut) to the layer count
            pattern = (pattern * (num_layers // len(pattern) + 1))[:num_layers]
        self.pattern = pattern
        self.layers = nn.ModuleList(_HybridLayer(k, self.config, dict(mamba or {}), dict(moe or {})) for k in pattern)
        self.norm = RMSNorm(self.config.hidden_size, self.config.rms_norm_eps)

    def new_cache(self) -> List[dict]:
        return [dict() for _ in self.layers]

    def forward(self, inputs_embeds: torch.Tensor, cache: Optional[List[dict]] = None) -> torch.Tensor:
        x = inputs_embeds
        B, T, _ = x.shape
        past = 0
        if cache is not None:
            past = int(cache[0].get("_pos", 0))
            cache[0]["_pos"] = past + T
        pos = torch.arange(past, past + T, device=x.device).unsqueeze(0).expand(B, T)
        cos, sin = rope_tables(pos, self.config.dh, self.config.rope_theta)
        for li, layer in enumerate(self.layers):
            x = layer(x, cos, sin, None, cache[li] if cache is not None else None)
        return self.norm(x)


class EasyMagpieTTSModel(ModelPT):
    """Batch: ``text`` [B, Lt], ``text_len`` [B], ``codes`` [B, C, Ta] (codec tokens), ``codes_len`` [B]."""

    def __init__(self, cfg: DictConfig, trainer=None, codec=None, tokenizer=None):
        super().__init__(cfg=cfg, trainer=trainer)
        cfg = self._cfg
        self.codec, self.tokenizer = codec, tokenizer
        self.C, self.N = int(cfg_get(cfg, "num_codebooks", 4)), int(cfg_get(cfg, "codebook_size", 64))
        self.audio_bos_id, self.audio_eos_id = self.N, self.N + 1
        self.vocab = self.N + 2
        self.backbone_type = str(cfg_get(cfg, "backbone_type", "transformer"))
        lcfg = dict(cfg.backbone)
        if self.backbone_type == "nemotron_h":
            self.backbone = NemotronHDecoder(LLMConfig(**lcfg), str(cfg_get(cfg, "hybrid_pattern", "M-M*-")), dict(cfg_get(cfg, "mamba", {}) or {}),
                                             dict(cfg_get(cfg, "moe", {}) or {}))
            hidden, text_vocab = self.backbone.config.hidden_size, self.backbone.config.vocab_size
        elif self.backbone_type == "transformer":
            self.backbone = CausalLM.from_config(lcfg)
            hidden, text_vocab = self.backbone.config.hidden_size, self.backbone.config.vocab_size
            self.backbone.model.embed_tokens = None
            self.backbone.lm_head = None
        else:
            raise ValueError("backbone_type must be 'transformer' or 'nemotron_h'")
        self.text_emb = nn.Embedding(text_vocab, hidden)
        self.audio_emb = nn.ModuleList(nn.Embedding(self.vocab, hidden) for _ in range(self.C))
        self.heads = nn.ModuleList(nn.Linear(hidden, self.vocab) for _ in range(self.C))
        if not self._is_model_being_restored and self._train_dl is None:
            self._setup_dataloaders_from_cfg()

    def _setup_dataloaders_from_cfg(self):
        if hasattr(self, "heads"):                                                       # the base constructor calls this before the layers exist
            super()._setup_dataloaders_from_cfg()

    def _loader(self, c):
        from .code_datasets import build_code_dataloader

        return build_code_dataloader(c, num_codebooks=self.C, codebook_size=self.N, text_vocab=self.text_emb.num_embeddings, tokenizer=self.tokenizer)

    def setup_training_data(self, c):
        self._train_dl = self._loader(c)

    def setup_validation_data(self, c):
        self._validation_dl = self._loader(c)

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        with torch.no_grad():
            logits, tgt, mask = self(batch["text"], batch["text_len"], batch["codes"].long(), batch["codes_len"])
        return {"val_loss": F.cross_entropy(logits[mask].reshape(-1, self.vocab), tgt[mask].reshape(-1))}

    # ------------------------------------------------------------------ pieces
    def _embed_frames(self, codes: torch.Tensor) -> torch.Tensor:
        """codes [B, C, T] -> [B, T, hidden]."""
        return sum(self.audio_emb[c](codes[:, c]) for c in range(self.C))

    def _run(self, x: torch.Tensor, cache=None, attention_mask=None) -> torch.Tensor:
        if self.backbone_type == "nemotron_h":
            return self.backbone(x, cache)
        return self.backbone(inputs_embeds=x, cache=cache, attention_mask=attention_mask, return_hidden=True)["hidden_states"]

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        return torch.stack([hd(h) for hd in self.heads], dim=-2).float()                    # [..., C, V]

    def forward(self, text, text_len, codes, codes_len):
        """Teacher forcing on left-aligned sequences ``text_b | BOS codes_b EOS``; returns (logits [B, Ta+1, C, V], targets, mask)."""
        B, C, Ta = codes.shape
        dev = codes.device
        bos = torch.full((B, C, 1), self.audio_bos_id, dtype=torch.long, device=dev)
        full = torch.cat([bos, codes, torch.full((B, C, 1), self.audio_eos_id, dtype=torch.long, device=dev)], dim=2)
        ar = torch.arange(Ta + 2, device=dev)
        full = torch.where((ar[None, None] == (codes_len + 1)[:, None, None]), torch.full_like(full, self.audio_eos_id), full)
        te, ae = self.text_emb(text), self._embed_frames(full[:, :, :-1])                   # audio inputs: BOS .. last code
        Lt = text.shape[1]
        # every utterance is packed as text_b then audio_b with no gap: right-pad the rest
        x = te.new_zeros(B, Lt + Ta + 1, te.shape[-1])
        pos_a = torch.zeros(B, Ta + 1, dtype=torch.long, device=dev)
        for b in range(B):
            lt = int(text_len[b])
            x[b, :lt] = te[b, :lt]
            x[b, lt:lt + Ta + 1] = ae[b]
            pos_a[b] = torch.arange(lt, lt + Ta + 1, device=dev)
        h = self._run(x)
        ha = h.gather(1, pos_a.unsqueeze(-1).expand(-1, -1, h.shape[-1]))
        targets = full[:, :, 1:].transpose(1, 2)                                            # [B, Ta+1, C]
        mask = ar[None, : Ta + 1] <= codes_len[:, None]                                     # the EOS frame is a target too
        return self._logits(ha), targets, mask

    def training_step(self, batch, batch_idx):
        logits, tgt, mask = self(batch["text"], batch["text_len"], batch["codes"].long(), batch["codes_len"])
        loss = F.cross_entropy(logits[mask].reshape(-1, self.vocab), tgt[mask].reshape(-1))
        self.log_dict({"train_loss": loss.detach()})
        return {"loss": loss}

    @torch.no_grad()
    def infer_batch(self, text: torch.Tensor, max_steps: int = 200, temperature: float = 0.7, topk: int = 0, generator=None):
        """One utterance per row (equal text lengths, or call per utterance): returns codes [B, C, T] and lengths [B]."""
        self.eval()
        B = text.shape[0]
        cache = self.backbone.new_cache() if self.backbone_type == "nemotron_h" else [dict() for _ in self.backbone.model.layers]
        bos = torch.full((B, self.C, 1), self.audio_bos_id, dtype=torch.long, device=text.device)
        x = torch.cat([self.text_emb(text), self._embed_frames(bos)], dim=1)
        done = torch.zeros(B, dtype=torch.bool, device=text.device)
        lens = torch.zeros(B, dtype=torch.long, device=text.device)
        out = []
        for _ in range(max_steps):
            lg = self._logits(self._run(x, cache)[:, -1])                                   # [B, C, V]
            lg[..., self.audio_bos_id] = float("-inf")
            lg[:, 1:, self.audio_eos_id] = float("-inf")                                    # only the first codebook can end the utterance
            if temperature <= 0:
                tok = lg.argmax(-1)
            else:
                if topk:
                    kth = lg.topk(min(topk, lg.shape[-1]), dim=-1).values[..., -1:]
                    lg = lg.masked_fill(lg < kth, float("-inf"))
                tok = torch.multinomial((lg / temperature).softmax(-1).view(-1, self.vocab), 1, generator=generator).view(B, self.C)
            done = done | (tok[:, 0] == self.audio_eos_id)
            if bool(done.all()):
                break
            lens = lens + (~done).long()
            out.append(tok.clamp(max=self.N - 1))
            x = self._embed_frames(tok.unsqueeze(-1))
        codes = torch.stack(out, dim=2) if out else torch.zeros(B, self.C, 0, dtype=torch.long, device=text.device)
        return codes, lens

    @torch.no_grad()
    def do_tts(self, transcript: str, **kw) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = torch.tensor([self.tokenizer.text_to_ids(transcript)], dtype=torch.long, device=self.text_emb.weight.device)
        codes, lens = self.infer_batch(ids, **kw)
        if self.codec is None:
            return codes, lens
        return self.codec.decode(tokens=codes, tokens_len=lens)
