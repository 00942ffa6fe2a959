"""CPU tests of the core layer: config tree, instantiation allow-list, neural types, schedulers, optimizers."""
import math
import os

import pytest
import torch

from speech_b200.core.config import DictConfig, MissingMandatoryValue, OmegaConf, apply_overrides, hydra_runner, open_dict
from speech_b200.core.instantiate import instantiate, locate
from speech_b200.core.neural_types import (AcousticEncodedRepresentation, AudioSignal, ChannelType, LengthsType, NeuralType,
                                           NeuralTypeComparisonResult, SpectrogramType, MelSpectrogramType, typecheck)
from speech_b200.core.optim import lr_scheduler as S
from speech_b200.core.optim.optimizers import AVAILABLE_OPTIMIZERS, get_optimizer, parse_optimizer_args


def test_config_interpolation_and_resolvers():
    cfg = OmegaConf.create({"a": {"b": 4, "c": "${a.b}"}, "d": "${multiply:${a.b},3}", "e": "x_${a.c}", "f": "${sum:1,2,3}",
                            "lst": [1, {"k": "${a.b}"}]})
    assert cfg.a.c == 4 and cfg.d == 12 and cfg.e == "x_4" and cfg.f == 6
    assert cfg.lst[1].k == 4
    plain = OmegaConf.to_container(cfg, resolve=True)
    assert plain["d"] == 12 and plain["lst"][1]["k"] == 4
    y = OmegaConf.to_yaml(cfg)
    again = OmegaConf.create(y)
    assert again.a.c == 4


def test_config_struct_missing_and_overrides(tmp_path):
    cfg = OmegaConf.create({"model": {"lr": 1e-3, "name": "???"}, "trainer": {"devices": 1}})
    with pytest.raises(MissingMandatoryValue):
        _ = cfg.model.name
    OmegaConf.set_struct(cfg, True)
    with pytest.raises(Exception):
        cfg.model.new_key = 1
    with open_dict(cfg):
        cfg.model.new_key = 1
    apply_overrides(cfg, ["model.lr=0.5", "+model.extra.k=[1,2]", "trainer.devices=8", "~model.new_key", "model.name=abc"])
    assert cfg.model.lr == 0.5 and cfg.model.extra.k == [1, 2] and cfg.trainer.devices == 8 and "new_key" not in cfg.model
    assert cfg.model.name == "abc"
    p = tmp_path / "c.yaml"
    OmegaConf.save(cfg, str(p))
    assert OmegaConf.load(str(p)) == cfg
    merged = OmegaConf.merge(cfg, {"model": {"lr": 2.0}, "z": 1})
    assert merged.model.lr == 2.0 and merged.z == 1 and merged.model.name == "abc"


def test_yaml_float_exponent():
    assert OmegaConf.create("lr: 1e-3").lr == pytest.approx(1e-3)


def test_hydra_runner(tmp_path):
    (tmp_path / "conf.yaml").write_text("model:\n  dim: 8\n  scale: ${multiply:${model.dim},2}\n")
    seen = {}

    @hydra_runner(config_path=str(tmp_path), config_name="conf")
    def main(cfg):
        seen["cfg"] = cfg
        return cfg.model.scale

    assert main(argv=["model.dim=16"]) == 32
    assert seen["cfg"].model.dim == 16


def test_instantiate_allow_list_and_alias():
    enc = instantiate({"_target_": "nemo.collections.asr.modules.ConvASRDecoder", "feat_in": 16, "num_classes": 5,
                       "vocabulary": list("abcde")})
    assert type(enc).__name__ == "ConvASRDecoder" and enc.num_classes_with_blank == 6
    with pytest.raises(ValueError):
        instantiate({"_target_": "os.system", "command": "true"})
    assert locate("torch.nn.Linear") is torch.nn.Linear


def test_neural_types_and_typecheck():
    a = NeuralType(("B", "D", "T"), SpectrogramType())
    b = NeuralType(("B", "D", "T"), MelSpectrogramType())
    assert a.compare(b) == NeuralTypeComparisonResult.GREATER and b.compare(a) == NeuralTypeComparisonResult.LESS
    assert a.compare(NeuralType(("B", "T", "D"), SpectrogramType())) == NeuralTypeComparisonResult.TRANSPOSE_SAME
    assert NeuralType(("B", "T"), AudioSignal(16000)).compare(NeuralType(("B", "T"), AudioSignal(8000))) == \
        NeuralTypeComparisonResult.SAME_TYPE_INCOMPATIBLE_PARAMS

    class M(torch.nn.Module):
        @property
        def input_types(self):
            return {"x": NeuralType(("B", "T"), ChannelType()), "n": NeuralType(("B",), LengthsType(), optional=True)}

        @property
        def output_types(self):
            return {"y": NeuralType(("B", "T"), ChannelType())}

        @typecheck()
        def forward(self, x, n=None):
            return x * 2

    m = M()
    out = m(x=torch.ones(2, 3))
    assert out.neural_type.elements_type.__class__ is ChannelType
    with pytest.raises(TypeError):
        m(torch.ones(2, 3))
    with pytest.raises(TypeError):
        m(x=torch.ones(2, 3, 4))
    with typecheck.disable_checks():
        m(torch.ones(2, 3))


def test_noam_and_cosine_schedules():
    p = [torch.nn.Parameter(torch.zeros(1))]
    opt = torch.optim.SGD(p, lr=2.0)
    sch = S.NoamAnnealing(opt, d_model=256, warmup_steps=100, min_lr=1e-6)
    lrs = []
    for _ in range(300):
        opt.step()
        sch.step()
        lrs.append(opt.param_groups[0]["lr"])
    step = 150
    expect = 2.0 * 256 ** -0.5 * min(step ** -0.5, step * 100 ** -1.5)
    assert lrs[step - 1] == pytest.approx(expect, rel=1e-6)
    assert max(lrs) == pytest.approx(2.0 * 256 ** -0.5 * 100 ** -0.5, rel=1e-6)
    opt = torch.optim.SGD(p, lr=1.0)
    cos = S.CosineAnnealing(opt, max_steps=100, warmup_steps=10, min_lr=0.1)
    vals = []
    for _ in range(100):
        opt.step()
        cos.step()
        vals.append(opt.param_groups[0]["lr"])
    assert vals[9] == pytest.approx(1.0, rel=1e-6)
    assert vals[-1] == pytest.approx(0.1, abs=1e-6)
    assert all(x >= y - 1e-9 for x, y in zip(vals[10:], vals[11:]))


def test_scheduler_registry_and_prepare():
    names = ["WarmupPolicy", "WarmupHoldPolicy", "SquareAnnealing", "CosineAnnealing", "NoamAnnealing", "NoamHoldAnnealing",
             "WarmupAnnealing", "InverseSquareRootAnnealing", "T5InverseSquareRootAnnealing", "SquareRootAnnealing",
             "PolynomialDecayAnnealing", "PolynomialHoldDecayAnnealing", "StepLR", "ExponentialLR", "ReduceLROnPlateau", "CyclicLR",
             "WarmupHoldAnnealOneMinusSquareRoot", "WarmupHoldAnnealLinear"]
    for n in names:
        assert n in S.AVAILABLE_SCHEDULERS
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    out = S.prepare_lr_scheduler(opt, {"name": "CosineAnnealing", "warmup_steps": 2, "max_steps": 10, "min_lr": 0.0})
    assert out["interval"] == "step" and isinstance(out["scheduler"], S.CosineAnnealing)


def test_optimizer_registry():
    for n in ["sgd", "adam", "adamw", "adadelta", "adamax", "adagrad", "rmsprop", "rprop", "novograd", "adafactor", "adan",
              "fused_adam"]:
        assert n in AVAILABLE_OPTIMIZERS
    kw = parse_optimizer_args("adamw", {"name": "adamw", "lr": 1e-3, "betas": [0.9, 0.98], "sched": {"name": "x"}})
    assert kw == {"lr": 1e-3, "betas": (0.9, 0.98)}
    w = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    for name in ("novograd", "adan", "adafactor"):
        kwargs = {"lr": 0.05} if name != "adafactor" else {"lr": 0.05, "relative_step": False, "scale_parameter": False}
        q = torch.nn.Parameter(w.detach().clone())
        opt = get_optimizer(name)([q], **kwargs)
        first = None
        for _ in range(30):
            opt.zero_grad()
            loss = (q ** 2).sum()
            first = first if first is not None else float(loss)
            loss.backward()
            opt.step()
        assert float((q ** 2).sum()) < first, name


def test_fused_adamw_cpu_matches_torch_and_fusion_views():
    from speech_b200.core.optim.fused_adamw import FusedAdamW

    torch.manual_seed(0)
    a, b, c = (torch.nn.Parameter(torch.randn(128, 16)) for _ in range(3))
    other = torch.nn.Parameter(torch.randn(7))
    ref = [torch.nn.Parameter(p.detach().clone()) for p in (a, other, b, c)]
    opt = FusedAdamW([a, other, b, c], lr=1e-2, betas=(0.9, 0.98), weight_decay=0.1, fusion_groups=[[a, b, c]])
    fused = opt.arena.fuse([a, b, c])
    assert fused is not None and fused.shape == (384, 16)
    assert fused.data_ptr() == a.data_ptr()
    topt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.98), weight_decay=0.1)
    for _ in range(4):
        opt.zero_grad()
        for p, r in zip((a, other, b, c), ref):
            g = torch.randn_like(p)
            p.grad.copy_(g)
            r.grad = g.clone()
        opt.step()
        topt.step()
    for p, r in zip((a, other, b, c), ref):
        assert torch.allclose(p, r, atol=1e-6)
    sd = opt.state_dict()
    opt.load_state_dict(sd)


def test_ema_optimizer_and_main_params_wrapper():
    import torch

    from speech_b200.core.optim.wrappers import EMAOptimizer, MainParamsOptimizerWrapper

    torch.manual_seed(0)
    lin = torch.nn.Linear(4, 3)
    opt = EMAOptimizer(torch.optim.SGD(lin.parameters(), lr=0.5), decay=0.5)
    w0 = lin.weight.detach().clone()
    lin(torch.ones(2, 4)).sum().backward()
    opt.step()
    w1 = lin.weight.detach().clone()
    assert torch.allclose(opt.ema_params[0], w1)            # first step: the average starts at the weights
    opt.zero_grad()
    lin(torch.ones(2, 4)).sum().backward()
    opt.step()
    w2 = lin.weight.detach().clone()
    assert torch.allclose(opt.ema_params[0], 0.5 * w1 + 0.5 * w2, atol=1e-6) and not torch.equal(w0, w2)
    with opt.swap_ema_weights():
        assert torch.allclose(lin.weight, 0.5 * w1 + 0.5 * w2, atol=1e-6)
    assert torch.equal(lin.weight, w2)
    sd = opt.state_dict()
    opt2 = EMAOptimizer(torch.optim.SGD(lin.parameters(), lr=0.5), decay=0.9)
    opt2.load_state_dict(sd)
    assert opt2.decay == 0.5 and opt2.current_step == 2 and torch.equal(opt2.ema_params[0], opt.ema_params[0])
    # bf16 model, fp32 main weights: tiny updates are not lost to bf16 rounding
    m = torch.nn.Linear(8, 8, bias=False).to(torch.bfloat16)
    with torch.no_grad():
        m.weight.fill_(1.0)
    wrap = MainParamsOptimizerWrapper(m.parameters(), lambda ps: torch.optim.SGD(ps, lr=1e-3), fp32_grad_accum=True)
    for _ in range(40):
        wrap.zero_grad()
        m(torch.ones(1, 8, dtype=torch.bfloat16)).sum().backward()
        assert m.weight.grad is None and float(wrap.main_params[0].grad.abs().sum()) > 0
        wrap.step()
    assert abs(float(wrap.main_params[0][0, 0]) - (1.0 - 40 * 1e-3)) < 1e-5 and abs(float(m.weight[0, 0]) - 0.96) < 0.004
    naive = torch.nn.Linear(8, 8, bias=False).to(torch.bfloat16)
    with torch.no_grad():
        naive.weight.fill_(1.0)
    o = torch.optim.SGD(naive.parameters(), lr=1e-3)
    for _ in range(40):
        o.zero_grad()
        naive(torch.ones(1, 8, dtype=torch.bfloat16)).sum().backward()
        o.step()
    assert float(naive.weight[0, 0]) == 1.0               # every update rounds away in bf16


def test_step_hooks_profiling_windows_and_scheduled_freezing(tmp_path):
    """nsys / memory windows call the profiler API on the configured steps and ranks only; freeze_updates freezes a
    sub-module for its scheduled updates and keeps it in train mode."""
    import torch
    from speech_b200.core.config import OmegaConf
    from speech_b200.core.profiling import StepHooks

    class Api:
        def __init__(self):
            self.calls = []
        def profiler_start(self): self.calls.append("start")
        def profiler_stop(self): self.calls.append("stop")
        def nvtx_push(self, n): self.calls.append("push")
        def nvtx_pop(self): self.calls.append("pop")
        def record_memory(self, on): self.calls.append(f"mem{int(on)}")
        def dump_memory(self, path): self.calls.append("dump"); open(path, "wb").write(b"x")

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.encoder = torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.Dropout(0.5))
            self.decoder = torch.nn.Linear(2, 2)

    cfg = OmegaConf.create({"nsys_profile": {"enabled": True, "start_step": 2, "end_step": 3, "ranks": [0]},
                            "memory_profile": {"enabled": True, "start_step": 1, "end_step": 1, "rank": 0, "output_path": str(tmp_path)},
                            "freeze_updates": {"enabled": True, "modules": {"encoder": 2, "decoder": [3, 4]}}})
    api, m = Api(), M().train()
    h = StepHooks(cfg, rank=0, cuda_api=api)
    frozen = []
    for step in range(6):
        h.batch_start(m, step, step)
        frozen.append((not m.encoder[0].weight.requires_grad, not m.decoder.weight.requires_grad))
        assert m.encoder.training
        h.batch_end(m, step, step + 1)
    assert frozen == [(True, False), (True, False), (False, True), (False, True), (False, False), (False, False)]
    assert api.calls == ["mem1", "dump", "mem0", "start", "push", "pop", "push", "pop", "stop"]
    assert (tmp_path / "memory_profile_rank0.pickle").exists()
    other = Api()
    h1 = StepHooks(cfg, rank=1, cuda_api=other)
    for step in range(5):
        h1.batch_start(m, step, step); h1.batch_end(m, step, step + 1)
    assert other.calls == []
    import pytest
    with pytest.raises(ValueError, match="end_step"):
        StepHooks(OmegaConf.create({"nsys_profile": {"enabled": True, "start_step": 5, "end_step": 1}}))
    with pytest.raises(ValueError, match="output_path"):
        StepHooks(OmegaConf.create({"memory_profile": {"enabled": True, "start_step": 0, "end_step": 1, "output_path": None}}))
    # execution-trace capture on CPU
    ch = StepHooks(OmegaConf.create({"chakra_profile": {"enabled": True, "start_step": 1, "end_step": 2, "warmup_steps": 0, "active_steps": 2,
                                                        "trace_dir": str(tmp_path)}}), rank=0, cuda_api=Api())
    for step in range(4):
        ch.batch_start(m, step, step)
        m.decoder(torch.randn(3, 2)).sum().backward()
        ch.batch_end(m, step, step + 1)
    import glob
    assert glob.glob(str(tmp_path / "*_chakra" / "rank-0.json"))


def test_model_catalogue_lists_by_class_and_resolves_names_from_the_local_cache(tmp_path, monkeypatch):
    from speech_b200.core import model_catalog as mc
    from speech_b200.models.ctc_models import EncDecCTCModel
    from speech_b200.models.rnnt_models import EncDecRNNTBPEModel

    names = [i.pretrained_model_name for i in EncDecRNNTBPEModel.list_available_models()]
    assert "parakeet-tdt-0.6b-v2" in names and "canary-1b" not in names
    assert all(i.location.startswith("https://") and i.class_ is EncDecRNNTBPEModel for i in EncDecRNNTBPEModel.list_available_models())
    assert [e.name for e in mc.search("sortformer")] == ["diar_sortformer_4spk-v1", "diar_streaming_sortformer_4spk-v2"]
    monkeypatch.setenv("NEMO_CACHE_DIR", str(tmp_path))
    assert mc.resolve_local("QuartzNet15x5Base-En") is None
    with pytest.raises(FileNotFoundError):
        EncDecCTCModel.from_pretrained("QuartzNet15x5Base-En")
    calls = []

    def downloader(url, dest):
        calls.append(url)
        open(dest, "wb").write(b"x")

    path = mc.fetch("QuartzNet15x5Base-En", downloader)
    assert mc.fetch("QuartzNet15x5Base-En", downloader) == path and len(calls) == 1 and "QuartzNet15x5Base-En" in calls[0]
    assert mc.resolve_local("QuartzNet15x5Base-En") == path


def test_trainer_manual_optimization_updates_each_optimizer_from_its_own_loss():
    import torch
    from speech_b200.core.config import OmegaConf
    from speech_b200.core.modelpt import ModelPT
    from speech_b200.core.trainer import Trainer

    class TwoPlayers(ModelPT):
        def __init__(self, cfg, trainer=None):
            super().__init__(cfg=cfg, trainer=trainer)
            self.a = torch.nn.Parameter(torch.tensor(1.0))
            self.b = torch.nn.Parameter(torch.tensor(1.0))
            self.automatic_optimization = False
            self.seen = []

        def setup_training_data(self, c):
            self._train_dl = torch.utils.data.DataLoader(torch.arange(4.0), batch_size=1)

        def setup_validation_data(self, c):
            self._validation_dl = None

        def configure_optimizers(self):
            self._optimizers = [torch.optim.SGD([self.a], lr=0.1), torch.optim.SGD([self.b], lr=0.1)]
            return self._optimizers

        def training_step(self, batch, batch_idx):
            tr = self._trainer
            assert tr.in_manual_step
            # player b minimises (a * b) with a held fixed; player a then minimises -(a * b) and its loss also reaches b
            tr.manual_step(self.a.detach() * self.b, self._optimizers[1])
            loss_a = -(self.a * self.b)
            tr.manual_step(loss_a, self._optimizers[0])
            self.seen.append((float(self.a), float(self.b)))
            return {"loss": loss_a.detach()}

    m = TwoPlayers(OmegaConf.create({"train_ds": {}}))
    m.setup_training_data(None)
    tr = Trainer(max_steps=1, accelerator="cpu", devices=1, enable_checkpointing=False, logger=False, gradient_clip_val=0.0)
    tr.fit(m)
    # b moved by -lr * a = 0.9 (its own loss only: the gradient that a's loss left on b was never applied); a moved by +lr * b
    assert tr.global_step == 1 and m.seen[0][1] == pytest.approx(0.9) and m.seen[0][0] == pytest.approx(1.0 + 0.1 * 0.9)


def test_trainer_resumes_bit_identically_from_a_dcp_directory(tmp_path):
    import torch
    from speech_b200.core.config import OmegaConf
    from speech_b200.core.modelpt import ModelPT
    from speech_b200.core.trainer import Trainer

    class Tiny(ModelPT):
        def __init__(self, cfg, trainer=None):
            super().__init__(cfg=cfg, trainer=trainer)
            torch.manual_seed(0)
            self.net = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.Tanh(), torch.nn.Linear(8, 1))

        def setup_training_data(self, c):
            g = torch.Generator().manual_seed(1)
            data = [(torch.randn(4, generator=g), torch.randn(1, generator=g)) for _ in range(12)]
            self._train_dl = torch.utils.data.DataLoader(data, batch_size=2, shuffle=False)

        def setup_validation_data(self, c):
            self._validation_dl = None

        def configure_optimizers(self):
            return torch.optim.Adam(self.net.parameters(), lr=1e-2)

        def training_step(self, batch, batch_idx):
            x, y = batch
            return {"loss": (self.net(x) - y).pow(2).mean()}

    def run(steps, ckpt=None):
        m = Tiny(OmegaConf.create({}))
        m.setup_training_data(None)
        tr = Trainer(max_steps=steps, accelerator="cpu", devices=1, enable_checkpointing=False, logger=False)
        tr.fit(m, ckpt_path=ckpt)
        return m, tr

    whole, _ = run(5)
    half, tr = run(3)
    path = str(tmp_path / "step3.dcp")
    tr.save_checkpoint(path)
    assert os.path.exists(os.path.join(path, ".metadata")) and os.path.exists(os.path.join(path, "trainer_state.pt"))
    resumed, tr2 = run(5, ckpt=path)
    assert tr2.global_step == 5
    for a, b in zip(whole.parameters(), resumed.parameters()):
        assert torch.equal(a, b)


def test_common_losses_datasets_and_metrics():
    import numpy as np
    import torch

    from speech_b200.data.concat import CodeSwitchedDataset, ConcatDataset, ConcatMapDataset, FallbackDataset
    from speech_b200.losses.extra import LatentSpeakerSupervisionLoss, MultiSimilarityLoss, SpanningLoss
    from speech_b200.utils.metrics import Perplexity, TopKClassificationAccuracy

    # speaker tokens 10, 11; words 1..5; pad 0
    labels = torch.tensor([[10, 1, 2, 11, 3, 10, 4, 0]])
    lss = LatentSpeakerSupervisionLoss([10, 11], pad_id=0, per_speaker_normalization=False)
    assert lss.active_speakers(labels).tolist() == [[0, 0, 0, 1, 1, 0, 0, 0]]
    V = 12
    good = torch.full((1, 8, V), -10.0)
    for t, s in enumerate([10, 10, 10, 11, 11, 10, 10, 10]):
        good[0, t, s] = 0.0
    bad = good.clone()
    bad[0, 4, 11], bad[0, 4, 10] = -10.0, 0.0                                # the word after <spk1> leans to speaker 0
    lg, lb = float(lss(torch.log_softmax(good, -1), labels)), float(lss(torch.log_softmax(bad, -1), labels))
    assert lg < 1e-3 and lb == pytest.approx(10.0 / 4, rel=1e-3)             # one of four word positions is wrong
    per = LatentSpeakerSupervisionLoss([10, 11], pad_id=0, per_speaker_normalization=True)
    assert float(per(torch.log_softmax(bad, -1), labels)) == pytest.approx(10.0 / 2, rel=1e-3)        # speaker 1 has one word: its error weighs a half
    with_ce = LatentSpeakerSupervisionLoss([10, 11], pad_id=0, include_ce_loss=True)
    assert float(with_ce(torch.log_softmax(good, -1), labels)) > lg
    torch.manual_seed(0)
    emb = torch.nn.Parameter(torch.randn(8, 4))
    y = torch.tensor([0, 0, 1, 1, 2, 2, 3, 3])
    ms = MultiSimilarityLoss()
    opt = torch.optim.Adam([emb], 0.05)
    first = float(ms(emb, y))
    for _ in range(60):
        opt.zero_grad()
        ms(emb, y).backward()
        opt.step()
    e = torch.nn.functional.normalize(emb.detach(), dim=-1)
    assert float(ms(emb, y)) < first and float((e[0] * e[1]).sum()) > float((e[0] * e[2]).sum())
    span_logits = torch.zeros(2, 5, 2)
    span_logits[0, 1, 0], span_logits[0, 3, 1] = 5.0, 5.0
    loss, s_, e_ = SpanningLoss()(span_logits, torch.tensor([1, 99]), torch.tensor([3, 99]))
    assert float(loss) < 0.1 and s_.shape == (2, 5)
    a, b = list(range(100, 110)), list(range(200, 203))
    rr = ConcatMapDataset([a, b], sampling_technique="round-robin")
    assert len(rr) == 20 and [rr[i] for i in range(4)] == [100, 200, 101, 201] and rr[7] == 200                 # the short one wraps around
    tmp = ConcatMapDataset([a, b], sampling_technique="temperature", sampling_temperature=1.0, seed=1)
    assert len(tmp) == 13 and 4 <= sum(x >= 200 for x in [tmp[i] for i in range(13)]) + 4 <= 12
    rnd = ConcatMapDataset([a, b], sampling_technique="random", sampling_probabilities=[0.0, 1.0])
    assert all(rnd[i] >= 200 for i in range(len(rnd)))
    parts = [list(ConcatDataset([a, b], sampling_technique="round-robin", global_rank=r, world_size=2)) for r in range(2)]
    assert len(parts[0]) == len(parts[1]) == 10 and sorted(parts[0] + parts[1]) == sorted([rr[i] for i in range(20)])
    mk = lambda base, n: [(torch.full((8000,), 0.01 * (base + 1)), torch.tensor(8000), torch.tensor([base, base]), torch.tensor(2)) for _ in range(n)]  # noqa: E731
    cs = CodeSwitchedDataset([mk(0, 6), mk(1, 6)], min_duration=1.0, max_duration=2.0, min_monolingual=0.0, pause_join=0.1, sample_rate=16000, return_lang_ids=True, seed=3)
    items = list(cs)
    assert items and all(1.0 <= (x[0].numel() / 16000) <= 2.3 for x in items[:-1]) and {int(v) for it in items for v in it[4]} == {0, 1}
    x0 = items[0]
    assert x0[2].numel() == x0[4].numel() and float(x0[0][:8000].pow(2).mean().sqrt()) == pytest.approx(10 ** (-25 / 20), rel=1e-3)

    class Flaky(torch.utils.data.Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            if i == 2:
                raise OSError("corrupt")
            return i

    fb = FallbackDataset(Flaky())
    assert [fb[i] for i in range(4)] == [0, 1, 1, 3] and fb.failures == 1
    acc = TopKClassificationAccuracy(top_k=[1, 2])
    acc.update(torch.tensor([[0.1, 0.7, 0.2], [0.5, 0.3, 0.2], [0.2, 0.3, 0.5]]), torch.tensor([1, 1, 0]))
    assert acc.compute() == [pytest.approx(1 / 3), pytest.approx(2 / 3)]
    ppl = Perplexity()
    ppl.update(probs=torch.full((2, 4), 0.25))
    ppl.update(logits=torch.tensor([[100.0, 0.0, 0.0, 0.0]]))
    assert ppl.compute() == pytest.approx((4 + 4 + 1) / 3, rel=1e-4)
    with pytest.raises(ValueError):
        Perplexity().update(probs=torch.full((1, 4), 0.3))


def test_optimizer_and_scheduler_param_records_and_config_builder():
    from dataclasses import dataclass

    import torch

    from speech_b200.core import config_schemas as S
    from speech_b200.core.optim.lr_scheduler import get_scheduler, register_scheduler
    from speech_b200.core.optim.optimizers import get_optimizer, register_optimizer

    cos = S.get_scheduler_config("CosineAnnealingParams", min_lr=1e-5)(max_steps=100, warmup_steps=10)
    assert cos.min_lr == 1e-5 and cos.max_steps == 100 and cos.last_epoch == -1
    w = torch.nn.Parameter(torch.zeros(2))
    opt = get_optimizer("novograd", **S.params_to_dict(S.get_optimizer_config("novograd", lr=0.1, weight_decay=0.01)))([w])
    assert opt.defaults["lr"] == 0.1 and tuple(opt.defaults["betas"]) == (0.95, 0.98)
    sched = get_scheduler("CosineAnnealing", **S.params_to_dict(cos))(opt)
    lrs = []
    for _ in range(12):
        opt.step(); sched.step(); lrs.append(sched.get_last_lr()[0])
    assert max(lrs) <= 0.1 + 1e-9 and lrs[0] < lrs[5] < lrs[9]
    assert "lr" not in S.params_to_dict(S.AdamParams()) and S.params_to_dict(S.AdamParams(lr=1.0))["betas"] == [0.9, 0.999]
    with pytest.raises(ValueError):
        S.get_scheduler_config("NopeParams")
    with pytest.raises(ValueError):
        S.get_optimizer_config("nope")
    assert S.get_optimizer_config(None, lr=1) == {"lr": 1}

    @dataclass
    class MySchedParams(S.SchedulerParams):
        k: int = 3

    class MySched(torch.optim.lr_scheduler.LRScheduler):
        def __init__(self, optimizer, k=3, last_epoch=-1):
            self.k = k
            super().__init__(optimizer, last_epoch)

        def get_lr(self):
            return [b / self.k for b in self.base_lrs]

    register_scheduler("MySchedForTest", MySched, MySchedParams)
    assert S.get_scheduler_config("MySchedParams", k=5)().k == 5
    with pytest.raises(ValueError):
        register_scheduler("MySchedForTest", MySched, MySchedParams)

    @dataclass
    class MyOptParams(S.OptimizerParams):
        momentum: float = 0.5

    register_optimizer("my_sgd_for_test", torch.optim.SGD, MyOptParams)
    assert S.params_to_dict(S.get_optimizer_config("my_sgd_for_test", lr=0.2)) == {"lr": 0.2, "momentum": 0.5}

    class Builder(S.ModelConfigBuilder):
        def _finalize_cfg(self):
            if self.model_cfg.train_ds is not None and self.model_cfg.validation_ds is None:
                self.model_cfg.validation_ds = S.DatasetConfig(batch_size=self.model_cfg.train_ds.batch_size, shuffle=False)

    b = Builder(S.ModelConfig())
    b.set_train_ds(S.DatasetConfig(batch_size=8, shuffle=True))
    b.set_optim(S.NovogradParams(lr=0.05), S.SchedConfig(name="CosineAnnealing", min_lr=1e-6))
    cfg = b.build()
    assert cfg.validation_ds.batch_size == 8 and cfg.optim.name == "novograd" and cfg.optim.lr == 0.05 and cfg.optim.sched.name == "CosineAnnealing"
    top = S.to_dictconfig(S.NemoConfig(name="exp", model=cfg))
    assert top.model.optim.sched.min_lr == 1e-6 and top.trainer.strategy == "ddp" and top.model.train_ds.shuffle is True and list(top.model.optim.betas) == [0.95, 0.98]
