"""CUDA-graph label-looping decode against the host-driven nested-loop implementation (same greedy decisions expected)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("loss,max_symbols", [("rnnt", 3), ("tdt", 10)])
def test_graph_decode_equals_host_loop(loss, max_symbols):
    from speech_b200.decoding.label_looping import GreedyBatchedLabelLoopingComputer
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    torch.manual_seed(3)
    m = EncDecRNNTBPEModel(fastconformer_transducer_config("small", vocab_size=24, loss=loss, dropout=0.0, n_layers=1, sched=None,
                                                           lr=1e-3, pred_rnn_layers=2)).cuda().eval()
    durations = [0, 1, 2, 3, 4] if loss == "tdt" else None
    blank = m.decoding.blank_id
    host = GreedyBatchedLabelLoopingComputer(m.decoder, m.joint, blank, durations, max_symbols, allow_cuda_graphs=False)
    graph = GreedyBatchedLabelLoopingComputer(m.decoder, m.joint, blank, durations, max_symbols, allow_cuda_graphs=True)
    x = torch.randn(5, 37, 176, device="cuda")
    lens = torch.tensor([37, 30, 12, 1, 25], device="cuda")
    h0, _, s0 = host(x, lens)
    h1, _, s1 = graph(x, lens)
    assert graph._graph is not None, "the graph path was not taken"
    assert torch.equal(h0.current_lengths, h1.current_lengths)
    for b in range(5):
        n = int(h0.current_lengths[b])
        assert torch.equal(h0.transcript[b, :n], h1.transcript[b, :n]), b
        assert torch.equal(h0.timestamps[b, :n], h1.timestamps[b, :n]), b
    assert torch.allclose(h0.scores, h1.scores, atol=1e-3)
    assert torch.equal(s0.time_jumps, s1.time_jumps) and torch.equal(s0.labels, s1.labels)
    # continuation over a second chunk from the returned state, and a second call reusing the captured graph
    x2 = torch.randn(5, 37, 176, device="cuda")
    a, _, _ = host(x2, lens, s0)
    b_, _, _ = graph(x2, lens, s1)
    assert torch.equal(a.current_lengths, b_.current_lengths)
    for b in range(5):
        n = int(a.current_lengths[b])
        assert torch.equal(a.transcript[b, :n], b_.transcript[b, :n])
