"""Decoder-only language model backbone (Qwen2 / Qwen3 / Llama shape) owned by the framework.

The reference builds its speech-LLMs on ``transformers.AutoModelForCausalLM`` (``speechlm2/models/salm.py:60-80``).  Here the
backbone is a native module whose projections run on the framework's tcgen05 GEMM (``ops.linear``) and whose parameter names
equal the Hugging Face checkpoint names (``model.layers.N.self_attn.q_proj.weight`` ...), so ``from_pretrained`` reads a
local HF directory (``config.json`` + ``*.safetensors`` / ``pytorch_model*.bin``) without any conversion step.

Features: RMSNorm, grouped-query attention with rotary position embedding, optional per-head q/k RMSNorm (Qwen3), SwiGLU
MLP, tied or separate output head, ``inputs_embeds`` entry (the embedding table can live outside the model, which the
speech-LLM relies on), KV-cache decoding with greedy / top-k / top-p sampling, packed (varlen) batches through a
block-diagonal causal mask, optional tensor parallelism (heads and MLP columns split over a process group).
"""
from __future__ import annotations

import glob
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


@dataclass
class LLMConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = True
    qk_norm: bool = True              # Qwen3; False for Llama / Qwen2
    attention_bias: bool = False      # True for Qwen2
    mlp_bias: bool = False
    model_type: str = "qwen3"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None
    # mixture of experts (Qwen3-MoE): 0 experts = dense model
    num_experts: int = 0
    num_experts_per_tok: int = 2
    moe_intermediate_size: Optional[int] = None
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    decoder_sparse_step: int = 1              # every n-th layer is sparse ...
    mlp_only_layers: tuple = ()               # ... except these, which stay dense

    @classmethod
    def from_hf(cls, d: Dict[str, Any]) -> "LLMConfig":
        mt = d.get("model_type", "llama")
        keys = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in keys}
        kw["qk_norm"] = mt in ("qwen3", "qwen3_moe")
        kw["attention_bias"] = d.get("attention_bias", mt == "qwen2")
        kw.setdefault("num_key_value_heads", d.get("num_attention_heads"))
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        if "num_local_experts" in d and "num_experts" not in d:         # Mixtral spelling
            kw["num_experts"] = d["num_local_experts"]
        if "mlp_only_layers" in kw:
            kw["mlp_only_layers"] = tuple(kw["mlp_only_layers"] or ())
        return cls(**kw)

    def is_sparse_layer(self, i: int) -> bool:
        return self.num_experts > 0 and i not in self.mlp_only_layers and (i + 1) % max(1, self.decoder_sparse_step) == 0

    @property
    def dh(self) -> int:
        return self.head_dim or self.hidden_size // self.num_attention_heads


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x):
        from ..ops.native_llm import rmsnorm

        return rmsnorm(x, self.weight, self.variance_epsilon)       # one kernel each way for bf16 on GPUs, fp32 PyTorch otherwise


def rope_tables(positions: torch.Tensor, dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = positions.float().unsqueeze(-1) * inv
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, H, T, D]; cos/sin: [B, T, D] (rotate-half convention of the HF implementations)."""
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return (x.float() * cos.unsqueeze(1) + rot.float() * sin.unsqueeze(1)).to(x.dtype)


class _Linear(nn.Linear):
    """``nn.Linear`` parameters, forward on the framework's GEMM."""

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class Attention(nn.Module):
    def __init__(self, cfg: LLMConfig, tp_size: int = 1):
        super().__init__()
        self.cfg, self.tp = cfg, tp_size
        dh = cfg.dh
        self.n_q, self.n_kv = cfg.num_attention_heads // tp_size, max(1, cfg.num_key_value_heads // tp_size)
        self.q_proj = _Linear(cfg.hidden_size, self.n_q * dh, bias=cfg.attention_bias)
        self.k_proj = _Linear(cfg.hidden_size, self.n_kv * dh, bias=cfg.attention_bias)
        self.v_proj = _Linear(cfg.hidden_size, self.n_kv * dh, bias=cfg.attention_bias)
        self.o_proj = _Linear(self.n_q * dh, cfg.hidden_size, bias=False)
        if cfg.qk_norm:
            self.q_norm = RMSNorm(dh, cfg.rms_norm_eps)
            self.k_norm = RMSNorm(dh, cfg.rms_norm_eps)

    def forward(self, x, cos, sin, attn_mask=None, cache: Optional[Dict[str, torch.Tensor]] = None, is_causal: bool = True):
        B, T, _ = x.shape
        dh = self.cfg.dh
        q = self.q_proj(x).view(B, T, self.n_q, dh)
        k = self.k_proj(x).view(B, T, self.n_kv, dh)
        v = self.v_proj(x).view(B, T, self.n_kv, dh)
        if self.cfg.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        from ..ops.native_llm import rope

        cos_c, sin_c = (cos if cos.shape[0] == B else cos.expand(B, -1, -1)).contiguous(), (sin if sin.shape[0] == B else sin.expand(B, -1, -1)).contiguous()
        q, k = rope(q, cos_c, sin_c), rope(k, cos_c, sin_c)        # on the [B, T, H, D] layout, before the head transpose
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        cp_gather = getattr(self, "cp_gather", None)
        if cp_gather is not None and cache is None:
            k, v = cp_gather(k), cp_gather(v)        # context parallelism: queries stay local, keys / values of all ranks
        if cache is not None:
            if "k" in cache:
                k = torch.cat([cache["k"], k], dim=2)
                v = torch.cat([cache["v"], v], dim=2)
            cache["k"], cache["v"] = k, v
        if self.n_kv != self.n_q:
            rep = self.n_q // self.n_kv
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        causal = is_causal and attn_mask is None and q.shape[2] == k.shape[2]
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=causal)
        return self.o_proj(o.transpose(1, 2).reshape(B, T, self.n_q * dh))


class MLP(nn.Module):
    def __init__(self, cfg: LLMConfig, tp_size: int = 1):
        super().__init__()
        inner = cfg.intermediate_size // tp_size
        self.gate_proj = _Linear(cfg.hidden_size, inner, bias=cfg.mlp_bias)
        self.up_proj = _Linear(cfg.hidden_size, inner, bias=cfg.mlp_bias)
        self.down_proj = _Linear(inner, cfg.hidden_size, bias=cfg.mlp_bias)

    def forward(self, x):
        from ..ops.native_llm import swiglu

        return self.down_proj(swiglu(self.gate_proj(x), self.up_proj(x)))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: LLMConfig, tp_size: int = 1, layer_idx: int = 0):
        super().__init__()
        self.self_attn = Attention(cfg, tp_size)
        if cfg.is_sparse_layer(layer_idx):
            from .moe import SparseMoEBlock

            self.mlp = SparseMoEBlock(cfg.hidden_size, cfg.moe_intermediate_size or cfg.intermediate_size, cfg.num_experts,
                                      cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.router_aux_loss_coef)
        else:
            self.mlp = MLP(cfg, tp_size)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.tp_reduce = None          # set by the tensor-parallel plan: all-reduce (or reduce-scatter) of partial sums

    def forward(self, x, cos, sin, attn_mask=None, cache=None):
        a = self.self_attn(self.input_layernorm(x), cos, sin, attn_mask, cache)
        if self.tp_reduce is not None:
            a = self.tp_reduce(a)
        x = x + a
        m = self.mlp(self.post_attention_layernorm(x))
        if self.tp_reduce is not None:
            m = self.tp_reduce(m)
        return x + m


class DecoderModel(nn.Module):
    def __init__(self, cfg: LLMConfig, tp_size: int = 1):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(cfg, tp_size, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)


class CausalLM(nn.Module):
    """``forward(input_ids | inputs_embeds, attention_mask, position_ids, cache)`` → dict(logits, cache)."""

    def __init__(self, cfg: LLMConfig, tp_size: int = 1):
        super().__init__()
        self.config = cfg
        self.model = DecoderModel(cfg, tp_size)
        self.lm_head = _Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.gradient_checkpointing = False
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def set_input_embeddings(self, emb):
        self.model.embed_tokens = emb

    @staticmethod
    def build_mask(attention_mask: Optional[torch.Tensor], T_q: int, T_k: int, dtype, device, seq_ids: Optional[torch.Tensor] = None,
                   q_offset: Optional[int] = None):
        """Additive mask [B, 1, T_q, T_k]: causal, key padding, and block-diagonal over ``seq_ids`` for packed batches.  The
        queries are positions ``q_offset .. q_offset + T_q`` of the key axis (default: the last ``T_q``)."""
        if attention_mask is None and seq_ids is None and q_offset is None:
            return None
        q0 = T_k - T_q if q_offset is None else q_offset
        i = torch.arange(q0, q0 + T_q, device=device).view(1, 1, T_q, 1)
        j = torch.arange(T_k, device=device).view(1, 1, 1, T_k)
        ok = j <= i
        if attention_mask is not None:
            ok = ok & attention_mask.bool().view(attention_mask.shape[0], 1, 1, T_k)
        if seq_ids is not None:
            ok = ok & (seq_ids.view(seq_ids.shape[0], 1, T_k, 1)[:, :, q0:q0 + T_q] == seq_ids.view(seq_ids.shape[0], 1, 1, T_k))
        # rows that can see nothing (left padding) attend to themselves to keep softmax finite
        ok = ok | (~ok.any(dim=-1, keepdim=True) & (j == i))
        return torch.zeros(ok.shape, dtype=dtype, device=device).masked_fill(~ok, float("-inf"))

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, position_ids=None, cache: Optional[List[dict]] = None,
                seq_ids: Optional[torch.Tensor] = None, return_hidden: bool = False, **_):
        if inputs_embeds is None:
            inputs_embeds = self.model.embed_tokens(input_ids)
        x = inputs_embeds
        cdt = ops.get_compute_dtype()
        if cdt is not None and x.dtype != cdt:
            x = x.to(cdt)
        B, T, _ = x.shape
        past = cache[0]["k"].shape[2] if cache and "k" in cache[0] else 0
        if position_ids is None:
            if attention_mask is not None:
                position_ids = (attention_mask.long().cumsum(-1) - 1).clamp(min=0)[:, -T:]
            else:
                position_ids = torch.arange(past, past + T, device=x.device).unsqueeze(0).expand(B, T)
        cp = getattr(self.model, "cp_group", None) if cache is None else None
        cp_slice = None
        if cp is not None:
            # context parallelism: this rank keeps a contiguous T / W slice of the sequence through every block; attention sees
            # the keys and values of all ranks (gathered inside each attention module)
            import torch.distributed as dist

            W, r = dist.get_world_size(cp), dist.get_rank(cp)
            if T % W:
                raise ValueError(f"sequence length {T} is not divisible by the context-parallel size {W}: pad the batch")
            Tl = T // W
            cp_slice = (r * Tl, (r + 1) * Tl)
            x = x[:, cp_slice[0]:cp_slice[1]]
            position_ids = position_ids[:, cp_slice[0]:cp_slice[1]]
        cos, sin = rope_tables(position_ids, self.config.dh, self.config.rope_theta)
        if cp_slice is not None:
            mask = self.build_mask(attention_mask, cp_slice[1] - cp_slice[0], T, x.dtype, x.device, seq_ids, q_offset=cp_slice[0])
        else:
            mask = self.build_mask(attention_mask, T, past + T, x.dtype, x.device, seq_ids)
        sp = getattr(self.model, "sp_scatter", None) is not None and cache is None
        if sp:
            # sequence parallelism: the residual stream lives as [B, T / W, H] between blocks (positions, mask and rotary tables
            # above refer to the full sequence, which the blocks see after their all-gather)
            x = self.model.sp_scatter(x)
        for li, layer in enumerate(self.model.layers):
            c = cache[li] if cache is not None else None
            if self.gradient_checkpointing and self.training and c is None:
                x = torch.utils.checkpoint.checkpoint(layer, x, cos, sin, mask, None, use_reentrant=False)
            else:
                x = layer(x, cos, sin, mask, c)
        x = self.model.norm(x)
        if sp:
            x = self.model.sp_gather(x)
        out = {"hidden_states": x, "cache": cache}
        if cp_slice is not None:
            out["cp_slice"] = cp_slice          # hidden states / logits cover these positions only
        if not return_hidden:
            out["logits"] = self.lm_head(x)
        return out

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, input_ids=None, inputs_embeds=None, attention_mask=None, max_new_tokens: int = 32, eos_token_id=None,
                 pad_token_id: Optional[int] = None, do_sample: bool = False, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, embed_fn=None) -> torch.Tensor:
        """Returns the newly generated ids [B, <= max_new_tokens] (left-padded prompts are supported through
        ``attention_mask``).  ``embed_fn`` maps token ids to embeddings when the table lives outside this module."""
        embed_fn = embed_fn or self.model.embed_tokens
        if inputs_embeds is None:
            inputs_embeds = embed_fn(input_ids)
        B = inputs_embeds.shape[0]
        dev = inputs_embeds.device
        eos = eos_token_id if eos_token_id is not None else self.config.eos_token_id
        eos_set = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else set())
        pad = pad_token_id if pad_token_id is not None else (self.config.pad_token_id if self.config.pad_token_id is not None else 0)
        cache = [dict() for _ in self.model.layers]
        mask = attention_mask if attention_mask is not None else torch.ones(inputs_embeds.shape[:2], dtype=torch.long, device=dev)
        out = self.forward(inputs_embeds=inputs_embeds, attention_mask=mask, cache=cache)
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        toks = []
        logits = out["logits"][:, -1].float()
        for _ in range(max_new_tokens):
            if do_sample:
                lg = logits / max(temperature, 1e-5)
                if top_k:
                    kth = lg.topk(min(top_k, lg.shape[-1]), dim=-1).values[:, -1:]
                    lg = lg.masked_fill(lg < kth, float("-inf"))
                if top_p < 1.0:
                    srt, idx = lg.sort(dim=-1, descending=True)
                    cum = srt.softmax(-1).cumsum(-1)
                    cut = cum - srt.softmax(-1) > top_p
                    srt = srt.masked_fill(cut, float("-inf"))
                    lg = torch.full_like(lg, float("-inf")).scatter(1, idx, srt)
                nxt = torch.multinomial(lg.softmax(-1), 1).squeeze(1)
            else:
                nxt = logits.argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            toks.append(nxt)
            for e in eos_set:
                done = done | (nxt == e)
            if bool(done.all()):
                break
            mask = torch.cat([mask, torch.ones((B, 1), dtype=mask.dtype, device=dev)], dim=1)
            out = self.forward(inputs_embeds=embed_fn(nxt.unsqueeze(1)), attention_mask=mask, cache=cache)
            logits = out["logits"][:, -1].float()
        return torch.stack(toks, dim=1) if toks else torch.zeros((B, 0), dtype=torch.long, device=dev)

    # ------------------------------------------------------------------ checkpoints
    @classmethod
    def from_config(cls, cfg: Any, **over) -> "CausalLM":
        if isinstance(cfg, LLMConfig):
            return cls(cfg)
        d = dict(cfg)
        d.update(over)
        return cls(LLMConfig.from_hf(d) if "model_type" in d else LLMConfig(**d))

    @classmethod
    def from_pretrained(cls, path: str, load_weights: bool = True, dtype=None, **over) -> "CausalLM":
        """``path``: a local Hugging Face model directory."""
        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        d.update(over)
        model = cls(LLMConfig.from_hf(d))
        if load_weights:
            sd: Dict[str, torch.Tensor] = {}
            files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
            if files:
                from safetensors.torch import load_file

                for fpath in files:
                    sd.update(load_file(fpath))
            else:
                for fpath in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
                    sd.update(torch.load(fpath, map_location="cpu", weights_only=True))
            if not sd:
                raise FileNotFoundError(f"no weight files (*.safetensors / pytorch_model*.bin) under {path}")
            if model.config.tie_word_embeddings:
                sd.pop("lm_head.weight", None)
            if model.config.num_experts > 0:
                from .moe import SparseMoEBlock

                for name, blk in model.named_modules():
                    if isinstance(blk, SparseMoEBlock) and f"{name}.experts.0.gate_proj.weight" in sd:
                        blk.load_per_expert(sd, prefix=name + ".")
                        for k in [k for k in sd if k.startswith(name + ".experts.") or k == name + ".gate.weight"]:
                            sd.pop(k)
                        sd[name + ".gate.weight"] = blk.gate.weight.detach()
                        sd[name + ".gate_up"], sd[name + ".down"] = blk.gate_up.detach(), blk.down.detach()
            missing, unexpected = model.load_state_dict(sd, strict=False)
            missing = [m for m in missing if not (m == "lm_head.weight" and model.config.tie_word_embeddings)]
            if missing:
                raise KeyError(f"missing weights: {missing[:8]}{'...' if len(missing) > 8 else ''}")
        if dtype is not None:
            model.to(dtype)
        return model

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        cfg = {k: getattr(self.config, k) for k in self.config.__dataclass_fields__}
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
        from safetensors.torch import save_file

        sd = {k: v.detach().cpu().contiguous() for k, v in self.state_dict().items()
              if not (k == "lm_head.weight" and self.config.tie_word_embeddings)}
        save_file(sd, os.path.join(path, "model.safetensors"))
