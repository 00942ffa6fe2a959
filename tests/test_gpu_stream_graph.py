"""Cache-aware encoder step replayed from a CUDA graph equals the eager step, with caches evolving over several chunks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_stream_step_graph_matches_eager():
    from speech_b200 import ops
    from speech_b200.modules.conformer_encoder import ConformerEncoder

    torch.manual_seed(0)
    enc = ConformerEncoder(feat_in=80, n_layers=3, d_model=256, n_heads=4, subsampling_factor=8, subsampling_conv_channels=64, conv_kernel_size=9,
                           causal_downsampling=True, conv_context_size="causal", att_context_size=[70, 1], att_context_style="chunked_limited",
                           conv_norm_type="layer_norm", dropout=0.0, dropout_att=0.0, dropout_pre_encoder=0.0, dropout_emb=0.0).cuda().eval()
    enc.setup_streaming_params()
    B = 6
    cfg = enc.streaming_cfg
    T = int(cfg.chunk_size[1] if isinstance(cfg.chunk_size, (list, tuple)) else cfg.chunk_size) + \
        int(cfg.pre_encode_cache_size[1] if isinstance(cfg.pre_encode_cache_size, (list, tuple)) else cfg.pre_encode_cache_size)
    chunks = [torch.randn(B, 80, T, device="cuda") for _ in range(4)]
    lens = torch.full((B,), T, device="cuda", dtype=torch.long)

    def run(graphs: bool):
        enc.stream_cuda_graphs = graphs
        enc.__dict__.pop("_stream_graphs", None)
        clc, clt, clcl = enc.get_initial_cache_state(batch_size=B, device="cuda")
        outs = []
        with torch.no_grad(), ops.compute_dtype(torch.bfloat16):
            for x in chunks:
                e, el, clc, clt, clcl = enc.cache_aware_stream_step(processed_signal=x, processed_signal_length=lens, cache_last_channel=clc,
                                                                      cache_last_time=clt, cache_last_channel_len=clcl, keep_all_outputs=False,
                                                                      drop_extra_pre_encoded=int(cfg.drop_extra_pre_encoded))
                clc, clt, clcl = clc.clone(), clt.clone(), clcl.clone()     # the graph hands out static buffers
                outs.append((e.float().clone(), el.clone()))
        torch.cuda.synchronize()
        return outs, (clc.float(), clt.float(), clcl)

    eager, ce = run(False)
    graphed, cg = run(True)
    assert len(enc._stream_graphs) == 1
    for (a, al), (b, bl) in zip(eager, graphed):
        assert torch.equal(al, bl) and torch.allclose(a, b, atol=2e-2, rtol=2e-2)
    assert torch.equal(ce[2], cg[2]) and torch.allclose(ce[0], cg[0], atol=2e-2) and torch.allclose(ce[1], cg[1], atol=2e-2)
    ops.native.check_status()
