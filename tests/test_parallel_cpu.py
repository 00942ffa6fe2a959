"""Parallel strategies on CPU (gloo, two ranks): device mesh, tensor-parallel LLM vs the unsharded model, vocabulary-
parallel cross entropy, sharded AdamW vs plain AdamW on averaged gradients, world-size independent optimizer checkpoints."""
import os
import subprocess
import sys
import textwrap

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.parallel.mesh import DeviceMesh
    from speech_b200.parallel.tp import apply_tensor_parallel_llm, vocab_parallel_cross_entropy
    from speech_b200.parallel.fsdp import ShardedFusedAdamW
    from speech_b200.core.optim.fused_adamw import FusedAdamW
    from speech_b200.speechlm.llm import CausalLM, LLMConfig
    mesh = DeviceMesh({{"tp": 2, "dp_shard": -1}})
    assert mesh.size("tp") == 2 and mesh.size("dp") == world // 2
    torch.manual_seed(0)
    cfg = LLMConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=8)
    ref = CausalLM(cfg); tp = CausalLM(cfg); tp.load_state_dict(ref.state_dict())
    apply_tensor_parallel_llm(tp, mesh.group("tp"))
    ids = torch.randint(0, 64, (2, 7))
    a = ref(input_ids=ids)["logits"]; b = tp(input_ids=ids)["logits"]
    assert torch.allclose(a, b, atol=1e-5), (a-b).abs().max()
    a.pow(2).mean().backward(); b.pow(2).mean().backward()
    g_ref = ref.model.layers[0].self_attn.q_proj.weight.grad.chunk(2, 0)[mesh.rank("tp")]
    assert torch.allclose(g_ref, tp.model.layers[0].self_attn.q_proj.weight.grad, atol=1e-6)
    assert torch.allclose(ref.model.embed_tokens.weight.grad, tp.model.embed_tokens.weight.grad, atol=1e-6)
    # sequence parallelism on top: residual stream sharded over the sequence, same logits and gradients
    from speech_b200.parallel.tp import allreduce_sequence_parallel_grads
    sp = CausalLM(cfg); sp.load_state_dict(ref.state_dict())
    apply_tensor_parallel_llm(sp, mesh.group("tp"), sequence_parallel=True)
    ids8 = torch.randint(0, 64, (2, 8))
    ref.zero_grad()
    a8 = ref(input_ids=ids8)["logits"]; c8 = sp(input_ids=ids8)["logits"]
    assert torch.allclose(a8, c8, atol=1e-5), (a8 - c8).abs().max()
    a8.pow(2).mean().backward(); c8.pow(2).mean().backward()
    allreduce_sequence_parallel_grads(sp, mesh.group("tp"))
    g_ref = ref.model.layers[1].mlp.down_proj.weight.grad.chunk(2, 1)[mesh.rank("tp")]
    assert torch.allclose(g_ref, sp.model.layers[1].mlp.down_proj.weight.grad, atol=1e-6)
    assert torch.allclose(ref.model.layers[0].input_layernorm.weight.grad, sp.model.layers[0].input_layernorm.weight.grad, atol=1e-6)
    assert torch.allclose(ref.model.norm.weight.grad, sp.model.norm.weight.grad, atol=1e-6)
    assert torch.allclose(ref.model.embed_tokens.weight.grad, sp.model.embed_tokens.weight.grad, atol=1e-6)
    # vocab-parallel CE
    lg = torch.randn(3, 5, 64); tg = torch.randint(0, 64, (3, 5)); tg[0, 0] = -100
    full = torch.nn.functional.cross_entropy(lg.view(-1, 64), tg.view(-1), ignore_index=-100, reduction="none").view(3, 5)
    dist.broadcast(lg, 0); dist.broadcast(tg, 0)
    full = torch.nn.functional.cross_entropy(lg.view(-1, 64), tg.view(-1), ignore_index=-100, reduction="none").view(3, 5)
    part = vocab_parallel_cross_entropy(lg.chunk(2, -1)[rank], tg, None)
    assert torch.allclose(full, part, atol=1e-5)
    # sharded AdamW == plain AdamW on averaged grads
    torch.manual_seed(1)
    def make():
        torch.manual_seed(1)
        return [torch.nn.Parameter(torch.randn(37, 5)), torch.nn.Parameter(torch.randn(300))]
    p1, p2 = make(), make()
    o1 = FusedAdamW(p1, lr=1e-2, max_grad_norm=1.0); o2 = ShardedFusedAdamW(p2, lr=1e-2, max_grad_norm=1.0)
    for it in range(3):
        torch.manual_seed(10 * it + rank)
        gs = [torch.randn_like(p) for p in p1]
        avg = [g.clone() for g in gs]
        for g in avg: dist.all_reduce(g); g.div_(world)
        for p, g in zip(p1, avg): p.grad.copy_(g)
        for p, g in zip(p2, gs): p.grad.copy_(g)
        o1.step(); o2.step()
        for a_, b_ in zip(p1, p2):
            assert torch.allclose(a_, b_, atol=1e-6), (it, (a_-b_).abs().max())
    sd = o2.state_dict()
    assert torch.allclose(sd["state"][0]["exp_avg"], o1.state_dict()["state"][0]["exp_avg"], atol=1e-7)
    o2.load_state_dict(sd)
    print("RESULT ok", rank)
    dist.destroy_process_group()
""")


def test_mesh_tp_and_sharded_optimizer_two_ranks(tmp_path):
    script = tmp_path / "par.py"
    script.write_text(SCRIPT.format(repo=REPO))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29762", str(script)],
                         capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stderr[-3000:]
    assert out.stdout.count("RESULT ok") == 2


def test_mesh_layout_without_process_groups():
    from speech_b200.parallel.mesh import DeviceMesh

    m = DeviceMesh({"dp_replicate": 2, "dp_shard": 2, "tp": 2}, rank=5, world_size=8, create_groups=False)
    assert m.coords == {"pp": 0, "dp_replicate": 1, "dp_shard": 0, "cp": 0, "tp": 1}
    assert m.ranks("tp") == [4, 5] and m.ranks("dp_shard") == [5, 7] and m.ranks("dp") == [1, 3, 5, 7]
    assert m.size("dp") == 4 and m.rank("dp") == 2 and not m.is_dp_source()


ORDER_SCRIPT = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.parallel.ddp import GradSync
    from speech_b200.core.modelpt import ModelPT

    # ---- (1) a parameter that is unused on one rank only: buckets must still pair up across ranks
    torch.manual_seed(0)
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Linear(8, 8); self.b = torch.nn.Linear(8, 8); self.c = torch.nn.Linear(8, 8)
        def forward(self, x, use_b):
            h = self.a(x)
            if use_b:
                h = h + self.b(x)
            return self.c(h).pow(2).mean()
    net = Net()
    # tiny buckets: every parameter tensor is its own bucket, so a wrong launch order would pair different tensors
    sync = GradSync(net, [], world, torch.device("cpu"), bucket_mb=1e-6)
    assert len(sync.buckets) >= 5
    launched = []
    orig = sync._launch
    def spy(bi):
        launched.append(bi); orig(bi)
    sync._launch = spy
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(100 + rank))
    for p in net.parameters():
        p.grad = None
    sync.begin_step()
    loss = net(x, use_b=(rank == 0))
    loss.backward()
    for p in net.b.parameters():        # the rank that skipped b contributes zeros
        if p.grad is None:
            p.grad = torch.zeros_like(p)
    sync.finish_step()
    assert launched == sorted(launched) and len(launched) == len(sync.buckets), launched
    # reference: plain average of the per-rank gradients
    ref = Net(); ref.load_state_dict(net.state_dict())
    ref(x, use_b=(rank == 0)).backward()
    for (n_, p), q in zip(net.named_parameters(), ref.parameters()):
        g = q.grad.clone() if q.grad is not None else torch.zeros_like(q)
        dist.all_reduce(g); g /= world
        assert torch.allclose(p.grad, g, atol=1e-6), n_

    # ---- (2) epoch-end metrics differ per rank before the reduction and agree after it
    from speech_b200.models.asr_model import ASRModel
    class Dummy:
        device = torch.device("cpu")
    outs = [{{"val_loss": torch.tensor(1.0 + rank), "val_wer_num": 3.0 + 5 * rank, "val_wer_denom": 10.0}}]
    res = ASRModel.multi_validation_epoch_end(type("M", (), {{"reduce_sums": staticmethod(ModelPT.reduce_sums), "device": torch.device("cpu")}})(), outs)
    assert abs(float(res["log"]["val_wer"]) - (3.0 + 8.0) / 20.0) < 1e-6, res
    assert abs(float(res["log"]["val_loss"]) - 1.5) < 1e-6, res
    # the generic path: any logged scalar becomes the mean over ranks
    m = type("M", (), {{"reduce_sums": staticmethod(ModelPT.reduce_sums), "device": torch.device("cpu")}})()
    synced = ModelPT._sync_logged(m, {{"val_acc": torch.tensor(0.25 + 0.5 * rank), "n": 2}})
    assert abs(float(synced["val_acc"]) - 0.5) < 1e-6
    print("RESULT ok", rank)
    dist.destroy_process_group()
""")


def test_bucket_order_and_metric_sync_two_ranks(tmp_path):
    """Buckets launch in index order even when gradients become final in a different order on one rank, and validation
    metrics are identical on all ranks after the epoch-end reduction."""
    script = tmp_path / "order.py"
    script.write_text(ORDER_SCRIPT.format(repo=REPO))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29764", str(script)],
                         capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stderr[-3000:]
    assert out.stdout.count("RESULT ok") == 2


FSDP2_SCRIPT = textwrap.dedent("""
    import os, sys, copy, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.parallel.fsdp2 import FullyShardedAdamW, FSDP2GradSync

    class Block(torch.nn.Module):
        def __init__(self, d):
            super().__init__()
            self.a = torch.nn.Linear(d, 2 * d); self.b = torch.nn.Linear(2 * d, d); self.n = torch.nn.LayerNorm(d)
        def forward(self, x):
            return x + self.b(torch.relu(self.a(self.n(x))))
    class Net(torch.nn.Module):
        def __init__(self, d=24, L=5):
            super().__init__()
            self.inp = torch.nn.Linear(7, d)
            self.layers = torch.nn.ModuleList(Block(d) for _ in range(L))
            self.head = torch.nn.Linear(d, 3)
        def forward(self, x):
            x = self.inp(x)
            for l in self.layers:
                x = l(x)
            return self.head(x)

    for clip in (0.0, 0.5):
        torch.manual_seed(0)
        ref = Net()
        net = copy.deepcopy(ref)
        ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=1e-2, betas=(0.9, 0.98))
        opt = FullyShardedAdamW(net, lr=1e-2, weight_decay=1e-2, betas=(0.9, 0.98), max_grad_norm=clip, device="cpu")
        sync = FSDP2GradSync(net, [opt], world, torch.device("cpu"))
        assert len(opt.units) == 5 and opt.root is not None
        rep = opt.memory_report()
        assert rep["persistent_fraction_of_replicated"] < 0.75      # tiny tensors: padding to 128 x W elements dominates
        # nothing replicated: layer parameters hold no data until their unit is gathered
        assert sum(p.numel() for l in net.layers for p in l.parameters()) <= 2 * max(u.numel for u in opt.units)
        for it in range(4):
            torch.manual_seed(100 * it + rank)
            x = torch.randn(6, 7); y = torch.randn(6, 3)
            # replicated reference: average of the ranks' gradients
            ref_opt.zero_grad()
            (ref(x) - y).pow(2).mean().backward()
            for p in ref.parameters():
                dist.all_reduce(p.grad); p.grad /= world
            if clip > 0:
                torch.nn.utils.clip_grad_norm_(ref.parameters(), clip)
            ref_opt.step()
            sync.begin_step()
            (net(x) - y).pow(2).mean().backward()
            sync.finish_step()
            opt.step()
            full = opt.gather_full_state()
            for (n_, pr), pn in zip(ref.named_parameters(), net.parameters()):
                assert torch.allclose(full[id(pn)], pr.detach(), atol=2e-6), (clip, it, n_, (full[id(pn)] - pr).abs().max())
        assert sync.launched_in_backward == 5
    # checkpoint round trip: full-by-name state written by two ranks continues identically in a fresh pair of ranks' objects
    import io
    model_sd, opt_sd = opt.full_model_state_dict(), opt.state_dict()
    assert set(model_sd) == set(ref.state_dict()) and all(tuple(model_sd[k].shape) == tuple(v.shape) for k, v in ref.state_dict().items())
    assert opt_sd["state"]["layers.2.a.weight"]["exp_avg"].shape == (48, 24) and opt_sd["step"] == 4
    buf = io.BytesIO(); torch.save({{"m": model_sd, "o": opt_sd}}, buf); buf.seek(0)
    ck = torch.load(buf, weights_only=False)
    torch.manual_seed(123)
    net2 = Net()                                       # different initial values: everything must come from the checkpoint
    opt2 = FullyShardedAdamW(net2, lr=1e-2, weight_decay=1e-2, betas=(0.9, 0.98), max_grad_norm=0.5, device="cpu")
    sync2 = FSDP2GradSync(net2, [opt2], world, torch.device("cpu"))
    opt2.load_full_params(ck["m"]); opt2.load_state_dict(ck["o"])
    for o_, s_, n_ in ((opt, sync, net), (opt2, sync2, net2)):
        torch.manual_seed(999 + rank)
        x = torch.randn(6, 7); y = torch.randn(6, 3)
        s_.begin_step(); (n_(x) - y).pow(2).mean().backward(); s_.finish_step(); o_.step()
    a, b = opt.gather_full_state(), opt2.gather_full_state()
    for pa, pb in zip(net.parameters(), net2.parameters()):
        assert torch.allclose(a[id(pa)], b[id(pb)], atol=1e-7), "resumed run diverges from the uninterrupted one"
    print("RESULT ok", rank)
    dist.destroy_process_group()
""")


def test_fully_sharded_adamw_matches_replicated_adamw_two_ranks(tmp_path):
    """ZeRO-3 units (gather before forward / backward, reduce-scatter + update after backward) against plain AdamW on averaged
    gradients, with and without global-norm clipping; parameters of ungathered units hold no data."""
    script = tmp_path / "fsdp2.py"
    script.write_text(FSDP2_SCRIPT.format(repo=REPO))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29766", str(script)],
                         capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1"))
    assert out.returncode == 0, out.stderr[-3000:]
    assert out.stdout.count("RESULT ok") == 2


SALM_MESH_SCRIPT = textwrap.dedent("""
    import os, sys, copy, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.core.config import OmegaConf
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.parallel.fsdp2 import FullyShardedAdamW, FSDP2GradSync
    from speech_b200.parallel.mesh import DeviceMesh
    from speech_b200.speechlm.data import SALMDataset, synthetic_conversations
    from speech_b200.speechlm.salm_automodel import SALMAutomodel
    from speech_b200.tokenizers import ByteLevelTokenizer

    TINY = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=8, tie_word_embeddings=False, qk_norm=True, model_type="qwen3")
    pc = {{"preprocessor": {{**preprocessor_cfg(32), "dither": 0.0}}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {{"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}, "output_dim": 32}}
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    cfg = OmegaConf.create({{"audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": TINY, "perception": pc,
                            "freeze_params": [], "prevent_freeze_params": [], "sequence_parallel": {sp}, "optim": {{"name": "adamw", "lr": 1e-3}}}})
    torch.manual_seed(0)
    ref = SALMAutomodel(cfg, tokenizer=tok).train()
    model = copy.deepcopy(ref)
    second = {second!r}
    mesh = DeviceMesh({{"dp_shard": 2, second: 2}})
    if second == "cp":
        from speech_b200.core.config import open_dict
        for mdl in (ref, model):
            with open_dict(mdl.cfg):
                mdl.cfg.packed_sequences = {{"enabled": True, "row_len": None}}
    model.configure_model(mesh)
    dp_rank, tp_rank = mesh.rank("dp_shard"), mesh.rank("tp")
    n_tp = sum(getattr(p, "_tensor_parallel", False) for p in model.parameters())
    assert (model._dp_size, n_tp > 0) == ((2, True) if second == "tp" else (4, False))
    kw = model._sharded_optimizer_kwargs()
    assert len(kw["units"]) == 3 and "replicate_group" not in kw
    opt = FullyShardedAdamW(model, lr=1e-2, weight_decay=0.0, max_grad_norm=0.3, device="cpu", **kw)
    if second == "tp":
        opt.set_tensor_parallel(mesh.group("tp"), lambda p: getattr(p, "_tensor_parallel", False))
    sync = FSDP2GradSync(model, [opt], opt.world, torch.device("cpu"))
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    ds = SALMDataset(synthetic_conversations(8, seed=3, min_duration=0.3, max_duration=0.6), tok, ref.prompt_formatter(), cfg.audio_locator_tag, ref.text_pad_id)
    for it in range(2):
        # data-parallel rank 0 gets one conversation, rank 1 gets three: very different numbers of labelled tokens
        parts = [[4 * it], [4 * it + 1, 4 * it + 2, 4 * it + 3]]
        batches = [ds.collate([ds[i] for i in p]) for p in parts]
        ref_opt.zero_grad()
        sums = [ref._token_loss_sums(b) for b in batches]
        n_total = sum(int(s[1]) for s in sums)
        (sum(s[0] for s in sums) / n_total).backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.3)
        ref_opt.step()
        sync.begin_step()
        out = model.training_step(batches[dp_rank], it)
        out["loss"].backward()
        model.on_after_backward()
        sync.finish_step()
        opt.step()
    full = opt.gather_full_state()
    worst = 0.0
    for (name, pr), pn in zip(ref.named_parameters(), model.parameters()):
        got, want = full[id(pn)], pr.detach()
        if getattr(pn, "_tensor_parallel", False):
            dim = [i for i, (a, b) in enumerate(zip(got.shape, want.shape)) if a != b][0]
            want = want.chunk(2, dim=dim)[tp_rank]
        err = float((got - want).abs().max())
        worst = max(worst, err)
        if name.endswith("depthwise_conv.bias"):
            continue          # a bias in front of batch norm has a zero gradient: Adam turns its rounding noise into steps
        assert err < 3e-4, (name, err)
    # validation sums are token weighted over the data-parallel group
    model.eval(); ref.eval()
    model.on_validation_epoch_start()
    with torch.no_grad():
        model.validation_step(batches[dp_rank], 0)
        model.on_validation_epoch_end()
    print("RESULT ok", rank, worst)
    dist.destroy_process_group()
""")


@pytest.mark.parametrize("sp,second", [(False, "tp"), (True, "tp"), (False, "cp")])
def test_salm_automodel_on_a_dp_shard_by_tp_or_cp_mesh_matches_single_process_four_ranks(tmp_path, sp, second):
    """2 (fully sharded data parallel) x 2 (tensor [+ sequence] parallel, or context parallel over packed sequences): after two
    steps with uneven labelled-token counts per data-parallel rank and global-norm clipping, every parameter slice equals the
    single-process model trained on the union of the batches with the per-token mean loss."""
    script = tmp_path / "salm_mesh.py"
    script.write_text(SALM_MESH_SCRIPT.format(repo=REPO, sp=sp, second=second))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                          "--master-addr", "127.0.0.1", "--master-port", str(29767 + int(sp) + 2 * (second == "cp")), str(script)],
                         capture_output=True, text=True, timeout=900, env=dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stderr[-4000:]
    assert out.stdout.count("RESULT ok") == 4


MOE_EP_SCRIPT = textwrap.dedent("""
    import os, sys, copy, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.speechlm.llm import CausalLM, LLMConfig
    from speech_b200.speechlm.moe import SparseMoEBlock, apply_expert_parallel, moe_aux_loss
    from speech_b200.parallel.ddp import GradSync
    from speech_b200.parallel.tp import apply_tensor_parallel_llm

    cfg = LLMConfig(vocab_size=48, hidden_size=16, intermediate_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=4,
                    num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8, router_aux_loss_coef=0.01, model_type="qwen3_moe",
                    tie_word_embeddings=False)
    torch.manual_seed(0)
    ref = CausalLM(cfg).train()
    ids_all = torch.randint(0, 48, (world, 3, 6))
    tgt_all = torch.randint(0, 48, (world, 3, 6))

    def loss_of(model, ids, tgt):
        lg = model(input_ids=ids)["logits"].float()
        l = torch.nn.functional.cross_entropy(lg.reshape(-1, 48), tgt.reshape(-1))
        aux = moe_aux_loss(model)
        return l + aux if aux is not None else l

    # ---- expert parallel x data parallel: rank r trains on batch r, experts are split
    ep = copy.deepcopy(ref)
    assert apply_expert_parallel(ep, dist.group.WORLD) == 2
    assert ep.model.layers[0].mlp.gate_up.shape[0] == 2
    sync = GradSync(ep, [], world, torch.device("cpu"))
    assert all(not getattr(p, "_no_dp_sync", False) for p in sync.params) and len(sync.params) < len(list(ep.parameters()))
    sync.begin_step() if hasattr(sync, "begin_step") else None
    loss_of(ep, ids_all[rank], tgt_all[rank]).backward()
    sync.finish_step()
    # single process: mean over the ranks' batches.  The auxiliary loss of the parallel model uses group-wide routing statistics,
    # so the reference computes it on the concatenated batch.
    ref.zero_grad()
    lg = ref(input_ids=ids_all.reshape(-1, 6))["logits"].float()
    ce = torch.nn.functional.cross_entropy(lg.reshape(-1, 48), tgt_all.reshape(-1))
    (ce + moe_aux_loss(ref)).backward()
    worst = 0.0
    for (n, pr), (_, pe) in zip(ref.named_parameters(), ep.named_parameters()):
        want = pr.grad
        if getattr(pe, "_expert_parallel", False):
            want = want[rank * 2:(rank + 1) * 2]
        err = float((pe.grad - want).abs().max()) / (float(want.abs().max()) + 1e-12)
        worst = max(worst, err)
        assert err < 2e-4, (n, err)
    # ---- tensor parallel over the experts' inner dimension: same batch on both ranks
    tp = copy.deepcopy(ref)
    tp.zero_grad()
    apply_tensor_parallel_llm(tp, dist.group.WORLD)
    assert tp.model.layers[0].mlp.gate_up.shape == (4, 8, 16)
    ids, tgt = ids_all[0], tgt_all[0]
    ref.zero_grad()
    l_ref = loss_of(ref, ids, tgt); l_ref.backward()
    l_tp = loss_of(tp, ids, tgt); l_tp.backward()
    assert abs(float(l_ref) - float(l_tp)) < 1e-5 + 0.01 * 0.5 * 2.5       # the parallel model reports aux / tp_size
    for (n, pr), (_, pt) in zip(ref.named_parameters(), tp.named_parameters()):
        want = pr.grad
        if getattr(pt, "_tensor_parallel", False):
            if n.endswith("gate_up"):
                want = want.view(4, 2, 8, 16).chunk(2, dim=2)[rank].reshape(4, 8, 16)
            else:
                dim = [i for i, (a, b) in enumerate(zip(pt.shape, want.shape)) if a != b][0]
                want = want.chunk(2, dim=dim)[rank]
        err = float((pt.grad - want).abs().max()) / (float(want.abs().max()) + 1e-12)
        assert err < 2e-4, ("tp", n, err)
    print("RESULT ok", rank, worst)
    dist.destroy_process_group()
""")


def test_moe_expert_parallel_and_expert_tensor_parallel_gradients_two_ranks(tmp_path):
    """Experts split over two ranks (dispatch / combine all-to-all) with data-parallel averaging of the dense parameters, and
    experts split along their inner dimension under tensor parallelism: every gradient equals the single-process one."""
    script = tmp_path / "moe_ep.py"
    script.write_text(MOE_EP_SCRIPT.format(repo=REPO))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29771", str(script)],
                         capture_output=True, text=True, timeout=600, env=dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stderr[-4000:]
    assert out.stdout.count("RESULT ok") == 2


def test_parallel_strategy_sizes_validation_and_sampler_arguments():
    from speech_b200.parallel.strategy import ParallelStrategy
    from speech_b200.speechlm.llm import LLMConfig

    st = ParallelStrategy(dp_replicate_size=2, dp_shard_size=-1, tp_size=2, sequence_parallel=True)
    mesh = st.setup(world_size=16, rank=5, create_groups=False)
    assert mesh.sizes == {"pp": 1, "dp_replicate": 2, "dp_shard": 4, "cp": 1, "tp": 2} and mesh.size("dp") == 8
    assert st.distributed_sampler_kwargs == {"num_replicas": 8, "rank": 2}            # rank 5 = (dp 2, tp 1)
    ok = LLMConfig(num_attention_heads=16, num_key_value_heads=8, intermediate_size=6144)
    assert st.validate(ok) == [] and st.validate(ok, max_sequence_multiple=8) == []
    bad = st.validate(LLMConfig(num_attention_heads=6, num_key_value_heads=3, intermediate_size=1001), max_sequence_multiple=3)
    assert len(bad) == 3 and "heads" in bad[0] and "feed-forward" in bad[1] and "multiples of 2" in bad[2]
    assert "sequence_parallel needs" in ParallelStrategy(tp_size=1, sequence_parallel=True).validate()[0]
    ep = ParallelStrategy(dp_shard_size=4, expert_parallel=True)
    ep.setup(world_size=4, rank=0, create_groups=False)
    assert "no experts" in ep.validate(ok)[0]
    assert "6 experts" in ep.validate(LLMConfig(num_attention_heads=4, num_key_value_heads=4, num_experts=6, moe_intermediate_size=64))[0]
    with pytest.raises(ValueError, match="pipeline"):
        ParallelStrategy(pp_size=2).setup(world_size=4, rank=0, create_groups=False)
    tp_only = ParallelStrategy(dp_shard_size=1, tp_size=4)
    tp_only.setup(world_size=4, rank=1, create_groups=False)
    assert tp_only.build_grad_sync(None, [], None) is None               # no rank sees different tokens: nothing to exchange


SALM_TRAINER_SCRIPT = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    from speech_b200.core.config import OmegaConf
    from speech_b200.core.trainer import Trainer
    from speech_b200.models.configs import encoder_cfg, preprocessor_cfg
    from speech_b200.parallel.strategy import ParallelStrategy
    from speech_b200.speechlm.salm_automodel import SALMAutomodel
    from speech_b200.tokenizers import ByteLevelTokenizer

    TINY = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=8, tie_word_embeddings=False, qk_norm=True, model_type="qwen3")
    pc = {{"preprocessor": {{**preprocessor_cfg(32), "dither": 0.0}}, "encoder": encoder_cfg("small", 32, 0.0, 0.0, n_layers=1),
          "modality_adapter": {{"_target_": "speech_b200.speechlm.perception.IdentityConnector", "d_model": 176}}}}
    tok = ByteLevelTokenizer(special_tokens=["<pad>", "<s>", "</s>", "<|im_start|>", "<|im_end|>"])
    def make():
        cfg = OmegaConf.create({{"audio_locator_tag": "<|audioplaceholder|>", "prompt_format": "qwen", "llm": TINY, "perception": pc,
                                "freeze_params": [], "prevent_freeze_params": [],
                                "train_ds": {{"synthetic": {{"num_samples": 16, "seed": 5, "min_duration": 0.3, "max_duration": 0.6}}, "batch_size": 2}},
                                "optim": {{"name": "fully_sharded_adamw", "lr": 1e-2, "weight_decay": 0.0}}}})
        torch.manual_seed(0)
        return SALMAutomodel(cfg, tokenizer=tok)
    ckpt = {ckpt!r}
    # run A: 4 steps in one go.  run B: 2 steps, checkpoint, fresh objects, 2 more steps from the checkpoint.
    def trainer(steps):
        return Trainer(max_steps=steps, accelerator="cpu", strategy=ParallelStrategy(dp_shard_size=2, tp_size=2), gradient_clip_val=0.5,
                       log_every_n_steps=1, enable_checkpointing=False, logger=False)
    ta = trainer(4); ma = make(); ta.fit(ma)
    rank = dist.get_rank()
    assert type(ta.grad_sync).__name__ == "FSDP2GradSync" and ma._dp_size == 2 and ta.global_step == 4
    assert len(ma._train_dl.ds) == 16 and ma._train_dl.world == 2                       # sharded over dp, not over all 4 ranks
    tb = trainer(2); mb = make(); tb.fit(mb)
    tb.save_checkpoint(ckpt)
    tc = trainer(4); mc = make(); tc.fit(mc, ckpt_path=ckpt)
    assert tc.global_step == 4
    fa, fc = ma._optimizer.gather_full_state(), mc._optimizer.gather_full_state()
    worst = max(float((fa[id(pa)] - fc[id(pc_)]).abs().max()) for pa, pc_ in zip(ma.parameters(), mc.parameters()))
    assert worst < 1e-5, worst
    print("RESULT ok", rank, worst)
    dist.destroy_process_group()
""")


def test_trainer_with_parallel_strategy_trains_salm_on_a_mesh_and_resumes_four_ranks(tmp_path):
    """Trainer(strategy=ParallelStrategy(dp_shard 2 x tp 2)) drives SALMAutomodel with the fully-sharded optimizer; a run that is
    check-pointed after two steps and resumed in fresh objects ends with the same parameters as the uninterrupted run."""
    script = tmp_path / "salm_trainer.py"
    script.write_text(SALM_TRAINER_SCRIPT.format(repo=REPO, ckpt=str(tmp_path / "step2.ckpt")))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                          "--master-addr", "127.0.0.1", "--master-port", "29773", str(script)],
                         capture_output=True, text=True, timeout=900, env=dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stderr[-4000:]
    assert out.stdout.count("RESULT ok") == 4


DCP_SCRIPT = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, {repo!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speech_b200.utils.dcp_io import DCPCheckpointIO
    path = {path!r}
    torch.manual_seed(0)
    table = torch.arange(10 * 3, dtype=torch.float32).view(10, 3)          # a row-sharded embedding: rank 0 holds 6 rows, rank 1 holds 4
    split = [(0, 6), (6, 4)][rank]
    replicated = torch.full((4,), 5.0)
    io = DCPCheckpointIO()
    io.save_checkpoint({{"emb": table[split[0]: split[0] + split[1]].clone(), "bias": replicated, "step": torch.tensor(11)}}, path,
                       sharded={{"emb": (split[0], 10)}}, extra={{"note": "two ranks"}})
    dist.barrier()
    # restore on the same two ranks with ANOTHER split (3 / 7 rows): every rank gets its new rows
    new = [(0, 3), (3, 7)][rank]
    tmpl = {{"emb": torch.zeros(new[1], 3), "bias": torch.zeros(4), "step": torch.tensor(0)}}
    out, extra = io.load_checkpoint(path, template=tmpl, sharded={{"emb": (new[0], 10)}})
    assert torch.equal(out["emb"], table[new[0]: new[0] + new[1]]) and torch.equal(out["bias"], replicated) and int(out["step"]) == 11
    assert extra == {{"note": "two ranks"}}
    dist.barrier()
    print("DCP_OK", rank)
""")


def test_dcp_checkpoint_written_by_two_ranks_reloads_with_another_sharding_and_on_one_rank(tmp_path):
    import torch

    from speech_b200.utils.dcp_io import DCPCheckpointIO

    script = tmp_path / "dcp_script.py"
    path = str(tmp_path / "ckpt")
    script.write_text(DCP_SCRIPT.format(repo=REPO, path=path))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29641",
                          str(script)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.count("DCP_OK") == 2, out.stderr[-3000:]
    state, extra = DCPCheckpointIO().load_checkpoint(path)                    # a single process reads the whole thing
    assert torch.equal(state["emb"], torch.arange(30, dtype=torch.float32).view(10, 3)) and int(state["step"]) == 11 and extra["note"] == "two ranks"
