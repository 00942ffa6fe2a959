"""SALM trained on a device mesh: fully-sharded / hybrid-sharded data parallelism, tensor + sequence parallelism, packed
batches and losses normalised by the global number of labelled tokens.

The reference gets these from ``nemo_automodel`` (``speechlm2/models/salm_automodel.py``: FSDP2 / HSDP / TP / SP plans,
packed THD batches ``parts/packed_sequences.py``, global-token normalisation ``:353-423``, validation sums ``:433-475``,
mesh-aware clipping ``:551-567``).  Here the pieces are this package's own:

* ``configure_model(mesh)`` applies the tensor-parallel plan (optionally sequence parallel) to the LLM over the mesh's ``tp``
  group and remembers the data-parallel groups;
* with ``optim.name: fully_sharded_adamw`` the parameters, gradients and AdamW state are sharded over ``dp_shard`` by
  :class:`speech_b200.parallel.fsdp2.FullyShardedAdamW` (units: every LLM block and every audio-encoder block; embeddings,
  output head and modality adapter form the root unit) and replicated over ``dp_replicate`` (hybrid sharding);
* mixture-of-experts LLMs (``speechlm/moe.py``) run expert parallel over the data-parallel group (``expert_parallel: true``)
  or with experts split along their inner dimension under ``tp``; the auxiliary load-balancing loss joins the training loss
  and ``moe_metrics`` logs expert loads;
* context parallelism (``cp``): each rank carries a slice of the (packed) sequence, attention gathers keys / values, and the
  ``cp`` ranks join the data-parallel ranks for loss normalisation and gradient averaging;
* ``pack_sequences`` turns a padded batch into rows without padding (several sequences per row, block-diagonal causal
  attention, positions restarting at every sequence);
* the training loss is ``sum of token losses on this rank x dp_size / labelled tokens of the whole data-parallel group``, so
  that the gradient average over data-parallel ranks is the gradient of the global per-token mean no matter how unevenly
  the labelled tokens are spread.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .salm import IGNORE_INDEX, SALM


def pack_sequences(input_embeds: torch.Tensor, attention_mask: torch.Tensor, target_ids: torch.Tensor,
                   row_len: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Padded ``[B, T, H]`` batch -> packed ``[R, L, H]`` rows.

    Sequences (the unpadded part of every row, wherever the padding sits) are placed first-fit in decreasing order of
    length into rows of capacity ``row_len`` (default: the total number of tokens, i.e. one row).  Returns
    ``input_embeds``, ``target_ids`` (``IGNORE_INDEX`` on padding), ``seq_ids`` (1-based sequence number per position, 0 on
    padding: attention is allowed only between equal ids), ``position_ids`` (restart at 0 in every sequence),
    ``attention_mask`` and ``cu_seqlens`` (``[R][n_r + 1]`` boundaries as a list of tensors)."""
    B, T, H = input_embeds.shape
    mask = attention_mask.bool()
    lens = mask.sum(dim=1).tolist()
    total = int(sum(lens))
    L = int(row_len or total)
    if max(lens) > L:
        raise ValueError(f"a sequence of {max(lens)} tokens does not fit rows of {L}")
    rows: List[List[int]] = []
    free: List[int] = []
    for b in sorted(range(B), key=lambda i: -lens[i]):
        if lens[b] == 0:
            continue
        for r in range(len(rows)):
            if free[r] >= lens[b]:
                rows[r].append(b)
                free[r] -= lens[b]
                break
        else:
            rows.append([b])
            free.append(L - lens[b])
    R = max(1, len(rows))
    emb = input_embeds.new_zeros((R, L, H))
    tgt = target_ids.new_full((R, L), IGNORE_INDEX)
    seq = torch.zeros((R, L), dtype=torch.long, device=input_embeds.device)
    pos = torch.zeros((R, L), dtype=torch.long, device=input_embeds.device)
    cu = []
    for r, members in enumerate(rows):
        o, bounds = 0, [0]
        for k, b in enumerate(members):
            n = lens[b]
            emb[r, o:o + n] = input_embeds[b][mask[b]]
            tgt[r, o:o + n] = target_ids[b][mask[b]]
            seq[r, o:o + n] = k + 1
            pos[r, o:o + n] = torch.arange(n, device=pos.device)
            o += n
            bounds.append(o)
        cu.append(torch.tensor(bounds, dtype=torch.int32, device=input_embeds.device))
    return {"input_embeds": emb, "target_ids": tgt, "seq_ids": seq, "position_ids": pos, "attention_mask": seq > 0, "cu_seqlens": cu}


class SALMAutomodel(SALM):
    """``cfg`` keys on top of SALM's: ``sequence_parallel`` (bool), ``packed_sequences: {enabled, row_len}``,
    ``expert_parallel`` (bool), ``moe_metrics: {enabled, mode, top_k_experts, every_n_steps}``."""

    def __init__(self, cfg, trainer=None, llm=None, tokenizer=None):
        super().__init__(cfg, trainer=trainer, llm=llm, tokenizer=tokenizer)
        self._device_mesh = None
        self._dp_group = None
        self._dp_size = 1
        self._val_sums: Dict[str, List[torch.Tensor]] = {}

    # ------------------------------------------------------------------ mesh
    @property
    def device_mesh(self):
        return self._device_mesh

    def configure_model(self, device_mesh=None) -> None:
        self._device_mesh = device_mesh
        if device_mesh is None:
            return
        from ..parallel.tp import apply_tensor_parallel_llm

        if device_mesh.size("pp") > 1:
            raise ValueError("pp > 1 is not available for SALMAutomodel; use dp_replicate / dp_shard / cp / tp")
        if device_mesh.size("tp") > 1:
            apply_tensor_parallel_llm(self.llm, device_mesh.group("tp"), sequence_parallel=bool(self.cfg.get("sequence_parallel", False)))
        if device_mesh.size("cp") > 1:
            from ..parallel.tp import apply_context_parallel_llm

            apply_context_parallel_llm(self.llm, device_mesh.group("cp"))
        # ranks that see different tokens: data parallel and context parallel alike (loss normalisation, gradient averaging)
        self._dp_size = device_mesh.size("dp_cp")
        self._dp_group = device_mesh.group("dp_cp") if self._dp_size > 1 else None
        if bool(self.cfg.get("expert_parallel", False)) and self._dp_group is not None:
            # experts are split over the data-parallel ranks; their gradients stay local, so the optimizer must keep
            # parameters per rank (no fully-sharded / arena optimizer for this model)
            from .moe import apply_expert_parallel

            if apply_expert_parallel(self.llm, self._dp_group) == 0:
                raise ValueError("expert_parallel is set but the LLM has no mixture-of-experts layers")
        self.setup_moe_options()
        # loaders built before the mesh existed were sharded over all ranks: rebuild them over the data-parallel group
        for attr, key in (("_train_dl", "train_ds"), ("_validation_dl", "validation_ds"), ("_test_dl", "test_ds")):
            if getattr(self, attr, None) is not None and self.cfg.get(key, None) is not None:
                setattr(self, attr, self._loader(self.cfg.get(key)))

    def setup_moe_options(self) -> None:
        """``moe_metrics: {enabled, mode: brief | detailed, top_k_experts, every_n_steps}`` switches expert-load tracking on."""
        mm = self.cfg.get("moe_metrics", None)
        if mm is not None and mm.get("enabled", False):
            from .moe import enable_load_tracking

            enable_load_tracking(self.llm, True)

    def maybe_log_moe_metrics(self, step: int) -> None:
        mm = self.cfg.get("moe_metrics", None)
        if mm is None or not mm.get("enabled", False) or step % int(mm.get("every_n_steps", 1)):
            return
        from .moe import collect_expert_loads, load_balance_summary

        loads = collect_expert_loads(self.llm, dp_group=self._dp_group)
        self.log_dict(load_balance_summary(loads))
        if mm.get("mode", "brief") == "detailed":
            k = int(mm.get("top_k_experts", 5))
            for name, v in loads.items():
                top = v.topk(min(k, v.numel()))
                self.log_dict({f"moe/{name}/expert_{int(i)}_load": float(x) for x, i in zip(top.values, top.indices)})

    def _sharded_optimizer_kwargs(self) -> Dict[str, Any]:
        m = self._device_mesh
        if any(getattr(p, "_expert_parallel", False) for p in self.parameters()):
            raise ValueError("expert-parallel experts differ per rank and cannot be sharded as replicas: use a per-rank optimizer "
                             "(for example optim.name: adamw with fused_optimizer: false)")
        kw: Dict[str, Any] = {"units": self.fsdp_units()}
        if m is not None:
            if m.size("dp_shard_cp") > 1:
                kw["group"] = m.group("dp_shard_cp")
            if m.size("dp_replicate") > 1:
                kw["replicate_group"] = m.group("dp_replicate")
        return kw

    def fsdp_units(self) -> List[torch.nn.Module]:
        """Modules gathered / resharded as one: each LLM block and each audio-encoder block.  What is left (embeddings, final
        norm, output head, modality adapter, pre-encoder) stays gathered for the whole step as the root unit."""
        units: List[torch.nn.Module] = []
        enc = getattr(self.perception, "encoder", None)
        if enc is not None and hasattr(enc, "layers"):
            units += list(enc.layers)
        units += list(self.llm.model.layers)          # forward order: backward meets (and reduces) them in reverse
        return [u for u in units if any(p.requires_grad for p in u.parameters())]

    def setup_optimization(self, optim_config=None, optim_kwargs=None):
        out = super().setup_optimization(optim_config, optim_kwargs)
        m = self._device_mesh
        opt = self._optimizer
        if m is not None and m.size("tp") > 1 and hasattr(opt, "set_tensor_parallel"):
            opt.set_tensor_parallel(m.group("tp"), lambda p: getattr(p, "_tensor_parallel", False))
        return out

    def configure_gradient_clipping(self, optimizer, gradient_clip_val: float) -> None:
        """Called by the trainer for optimizers that do not clip inside their own update."""
        from ..parallel.tp import clip_grad_norm_mesh

        m = self._device_mesh
        tp = m.group("tp") if m is not None and m.size("tp") > 1 else None
        params = [p for g in optimizer.param_groups for p in g["params"]]
        self._last_grad_norm = clip_grad_norm_mesh(params, gradient_clip_val, tp_group=tp)

    def on_after_backward(self):
        m = self._device_mesh
        if m is not None and m.size("tp") > 1 and bool(self.cfg.get("sequence_parallel", False)):
            from ..parallel.tp import allreduce_sequence_parallel_grads

            allreduce_sequence_parallel_grads(self.llm, m.group("tp"))

    def _loader(self, config):
        """Data is sharded over the ranks that must see different samples (the mesh's ``dp`` group); tensor- and
        context-parallel peers of a rank build the same batches from the same shard."""
        m = getattr(self, "_device_mesh", None)          # loaders are first built inside the base constructor
        if config is None or m is None:
            return super()._loader(config)
        from .data import build_salm_dataloader

        dp = m.size("dp")
        return build_salm_dataloader(config, self.tokenizer, self.prompt_formatter(), self.audio_locator_tag, self.text_pad_id,
                                     m.rank("dp") if dp > 1 else 0, dp)

    def _sequence_multiple(self) -> int:
        m = self._device_mesh
        if m is None:
            return 1
        mult = m.size("cp")
        if m.size("tp") > 1 and bool(self.cfg.get("sequence_parallel", False)):
            mult *= m.size("tp")
        return mult

    # ------------------------------------------------------------------ loss
    def _token_loss_sums(self, batch) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Dict[str, torch.Tensor]]:
        """(sum of token losses, number of labelled tokens, number predicted correctly, the model inputs)."""
        inp = self.prepare_inputs(batch)
        pk = self.cfg.get("packed_sequences", None)
        if pk is not None and pk.get("enabled", False):
            row_len = pk.get("row_len", None)
            mult = self._sequence_multiple()
            if row_len is None and mult > 1:
                total = int(inp["attention_mask"].sum())
                row_len = (total + mult - 1) // mult * mult
            packed = pack_sequences(inp["input_embeds"], inp["attention_mask"], inp["target_ids"], row_len)
            out = self.llm(inputs_embeds=packed["input_embeds"], attention_mask=packed["attention_mask"],
                           position_ids=packed["position_ids"], seq_ids=packed["seq_ids"], return_hidden=True)
            tgt = packed["target_ids"]
            inp = {**inp, "packed": packed}
        else:
            emb, am, tgt = inp["input_embeds"], inp["attention_mask"], inp["target_ids"]
            mult = self._sequence_multiple()
            if emb.shape[1] % mult:
                # sequence parallelism splits the time axis evenly over the tensor-parallel ranks: right-pad to a multiple
                extra = mult - emb.shape[1] % mult
                emb = F.pad(emb, (0, 0, 0, extra))
                am = F.pad(am, (0, extra), value=0)
                tgt = F.pad(tgt, (0, extra), value=IGNORE_INDEX)
            out = self.llm(inputs_embeds=emb, attention_mask=am, return_hidden=True)
        if "cp_slice" in out:
            tgt = tgt[:, out["cp_slice"][0]:out["cp_slice"][1]]        # this rank scores its slice of the sequence
        h = out["hidden_states"]
        labelled = tgt != IGNORE_INDEX
        n = labelled.sum()
        cap = batch.get("num_loss_tokens", None) if isinstance(batch, dict) else None
        if isinstance(cap, int) and 0 < cap < labelled.numel() // 2:
            # The output head runs on the labelled positions only (prompt and audio positions carry no target; with a 150 k-entry
            # vocabulary the head and the soft-max over every position are a sizeable part of the step).  ``num_loss_tokens`` is
            # an upper bound counted on the host when the batch was collated, so the selection needs no device-to-host read:
            # the first ``cap`` entries of a stable sort by the label flag; surplus entries are unlabelled and ignored by the loss.
            order = torch.argsort(labelled.reshape(-1).to(torch.uint8), descending=True, stable=True)[:cap]
            hs = h.reshape(-1, h.shape[-1]).index_select(0, order)
            ts = tgt.reshape(-1).index_select(0, order)
            logits = self.llm.lm_head(hs).float()
        else:
            logits = self.llm.lm_head(h).float()
            logits, ts = logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1)
        loss_sum = F.cross_entropy(logits, ts, ignore_index=IGNORE_INDEX, reduction="sum")
        correct = ((logits.argmax(dim=-1) == ts) & (ts != IGNORE_INDEX)).sum()
        return loss_sum, n, correct, inp

    def training_step(self, batch, batch_idx):
        loss_sum, n, _, inp = self._token_loss_sums(batch)
        n_global = n.clone()
        if self._dp_group is not None:
            dist.all_reduce(n_global, group=self._dp_group)
        n_global = n_global.clamp(min=1)
        # gradients are averaged over the dp ranks afterwards: dp_size x local sum / global count makes that average the
        # gradient of (sum over all ranks) / (labelled tokens on all ranks)
        loss = loss_sum * self._dp_size / n_global
        from .moe import moe_aux_loss

        aux = moe_aux_loss(self.llm)
        if aux is not None:
            loss = loss + aux
        self.maybe_log_moe_metrics(batch_idx)
        emb = inp["packed"]["input_embeds"] if "packed" in inp else inp["input_embeds"]
        B, T = emb.shape[:2]
        self.log_dict({"train_loss": (loss_sum.detach() / n.clamp(min=1)), "learning_rate": 0.0, "batch_size": float(B),
                       "sequence_length": float(T), "num_frames": float(n), "num_frames_global": float(n_global),
                       "target_to_input_ratio": float(n) / max(1, B * T)})
        return {"loss": loss}

    def on_validation_epoch_start(self):
        self._val_sums = {}

    def validation_step(self, batch, batch_idx, dataloader_idx=0):
        loss_sum, n, correct, _ = self._token_loss_sums(batch)
        sums = torch.stack([loss_sum.detach().double(), correct.double(), n.double()])
        self._val_sums.setdefault(str(dataloader_idx), []).append(sums)
        return {"val_loss": loss_sum.detach() / n.clamp(min=1)}

    def on_validation_epoch_end(self):
        """Token-weighted loss and accuracy over every rank's validation batches (sums are reduced, not means)."""
        names = sorted(self._val_sums)
        if self._dp_group is not None:
            # ranks may hold different subsets of loaders: agree on the list first
            gathered: List[Any] = [None] * self._dp_size
            dist.all_gather_object(gathered, names, group=self._dp_group)
            names = sorted({n for g in gathered for n in g})
        losses = []
        for name in names:
            parts = self._val_sums.get(name)
            dev = self.device
            s = torch.stack(parts).sum(dim=0) if parts else torch.zeros(3, dtype=torch.float64, device=dev)
            if self._dp_group is not None:
                s = s.to(dev)
                dist.all_reduce(s, group=self._dp_group)
            nf = s[2].clamp(min=1)
            tag = "" if len(names) == 1 else f"_{name}"
            self.log(f"val_loss{tag}", (s[0] / nf).float())
            self.log(f"val_acc{tag}", (s[1] / nf).float())
            losses.append(s[0] / nf)
        if len(names) > 1:
            self.log("val_loss", torch.stack(losses).mean().float())
        self._val_sums = {}
