"""Decoding extras on CPU: n-gram LM automaton, boosting tree, batched CTC prefix beam search, batched MALSD beam."""
import itertools
import math

import pytest
import torch

from speech_b200.decoding.batched_beam import BatchedBeamCTCComputer, ModifiedALSDBatchedComputer
from speech_b200.decoding.context_biasing import GPUBiasingMultiModel, GPUBoostingTreeModel, ctc_word_spotter
from speech_b200.decoding.ngram_lm import DEFAULT_TOKEN_OFFSET, NGramGPULanguageModel, write_arpa
from speech_b200.utils.streaming_utils import lcs_alignment_merge_buffer, longest_common_subsequence_merge

LN10 = math.log(10.0)


def _c(i):
    return chr(i + DEFAULT_TOKEN_OFFSET)


def test_ngram_lm_matches_bruteforce_backoff(tmp_path):
    V = 4
    grams = {("<s>",): (-99.0, -0.3), ("</s>",): (-1.0, 0.0), ("<unk>",): (-2.0, 0.0)}
    for i in range(V):
        grams[(_c(i),)] = (-0.5 - 0.1 * i, -0.2 - 0.05 * i)
    grams[(_c(0), _c(1))] = (-0.2, -0.4)
    grams[(_c(1), _c(2))] = (-0.3, -0.1)
    grams[("<s>", _c(0))] = (-0.25, -0.15)
    grams[(_c(0), _c(1), _c(2))] = (-0.05, 0.0)
    grams[(_c(1), _c(2), "</s>")] = (-0.6, 0.0)
    path = str(tmp_path / "lm.arpa")
    write_arpa(path, grams)
    lm = NGramGPULanguageModel.from_arpa(path, vocab_size=V)

    def brute(ctx, w):                       # ctx, w: tuples of ARPA words
        ctx = ctx[-2:]
        while True:
            if ctx + (w,) in grams:
                return grams[ctx + (w,)][0]
            if not ctx:
                return grams[("<unk>",)][0]
            bo = grams[ctx][1] if ctx in grams else 0.0
            return bo + brute(ctx[1:], w)

    for seq in itertools.product(range(V), repeat=3):
        st = lm.get_init_states(1, bos=True)
        ctx = ("<s>",)
        for t in seq:
            sc, nx = lm.advance(st)
            want = torch.tensor([brute(ctx, _c(v)) * LN10 for v in range(V)])
            assert torch.allclose(sc[0], want, atol=1e-5), (seq, ctx)
            st = nx[:, t]
            ctx = ctx + (_c(t),)
    lm.save_to(str(tmp_path / "lm.pt"))
    again = NGramGPULanguageModel.restore_from(str(tmp_path / "lm.pt"))
    assert abs(again.score_sentence([0, 1, 2]) - lm.score_sentence([0, 1, 2])) < 1e-6
    # p(0|<s>) + [backoff(<s> 0) + p(1|0)] + p(2|0 1)
    assert abs(lm.score_sentence([0, 1, 2]) - (-0.25 - 0.15 - 0.2 - 0.05) * LN10) < 1e-5


def test_boosting_tree_rewards_complete_phrases_only():
    tree = GPUBoostingTreeModel(vocab_size=8, phrases=[[1, 2, 3], [2, 4]], context_score=1.0)

    def walk(seq):
        st = tree.get_init_states(1)
        total = 0.0
        for t in seq:
            sc, nx = tree.advance(st)
            total += float(sc[0, t])
            st = nx[:, t]
        return total + float(tree.get_final(st)[0])

    assert walk([1, 2, 3]) == pytest.approx(3.0)
    assert walk([1, 2, 5]) == pytest.approx(0.0)         # partial match gives the reward back
    assert walk([1, 2, 4]) == pytest.approx(2.0)         # falls over to the second phrase through the failure link
    assert walk([1, 2]) == pytest.approx(0.0)            # unfinished at end of utterance
    assert walk([5, 2, 4, 6]) == pytest.approx(2.0)
    multi = GPUBiasingMultiModel(8)
    a = multi.add_model(tree, alpha=2.0)
    sc, _ = multi.advance(torch.zeros(2, dtype=torch.long), torch.tensor([a, -1]))
    assert float(sc[0, 1]) == 2.0 and float(sc[1].abs().sum()) == 0.0


def test_batched_ctc_beam_finds_best_labelling():
    torch.manual_seed(0)
    B, T, V = 3, 5, 3                                     # 2 labels + blank (index 2)
    lp = torch.log_softmax(torch.randn(B, T, V) * 2, dim=-1)
    lens = torch.tensor([5, 4, 3])
    beams = BatchedBeamCTCComputer(blank_index=2, beam_size=16)(lp, lens)
    got = beams.to_hyps_list(score_norm=False)
    for b in range(B):
        probs = {}
        for path in itertools.product(range(V), repeat=int(lens[b])):
            p = sum(float(lp[b, t, s]) for t, s in enumerate(path))
            lab, prev = [], 2
            for s in path:
                if s != prev and s != 2:
                    lab.append(s)
                prev = s
            probs[tuple(lab)] = math.log(math.exp(probs[tuple(lab)]) + math.exp(p)) if tuple(lab) in probs else p
        best = max(probs, key=probs.get)
        assert tuple(got[b][0][0]) == best
        assert got[b][0][2] == pytest.approx(probs[best], abs=1e-2)   # pruned prefixes take a little mass with them


def test_malsd_beam_one_equals_greedy_and_wider_beam_is_not_worse():
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    torch.manual_seed(1)
    m = EncDecRNNTBPEModel(fastconformer_transducer_config("small", vocab_size=16, loss="rnnt", dropout=0.0, n_layers=1,
                                                           sched=None, lr=1e-3))
    m.eval()
    enc = torch.randn(2, 7, m.joint.enc.in_features if hasattr(m.joint, "enc") else 176)
    lens = torch.tensor([7, 5])
    greedy = m.decoding.rnnt_decoder_predictions_tensor(enc.transpose(1, 2), lens, return_hypotheses=True)
    blank = m.decoding.blank_id
    k1 = ModifiedALSDBatchedComputer(m.decoder, m.joint, blank, beam_size=1, max_symbols_per_step=10)(enc, lens)
    h1 = k1.to_hyps_list(score_norm=False)
    for b in range(2):
        assert h1[b][0][0] == greedy[b].y_sequence.tolist()
    k4 = ModifiedALSDBatchedComputer(m.decoder, m.joint, blank, beam_size=4, max_symbols_per_step=10)(enc, lens)
    h4 = k4.to_hyps_list(score_norm=False)
    for b in range(2):
        assert max(s for _, _, s in h4[b]) >= h1[b][0][2] - 1e-4


@pytest.mark.parametrize("loss", ["rnnt", "tdt"])
def test_malsd_continues_a_stream_chunk_by_chunk_with_a_carry(loss):
    from speech_b200.decoding.batched_beam import MALSDCarry
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    torch.manual_seed(2)
    m = EncDecRNNTBPEModel(fastconformer_transducer_config("small", vocab_size=16, loss=loss, dropout=0.0, n_layers=1, sched=None, lr=1e-3)).eval()
    durations = [0, 1, 2, 3, 4] if loss == "tdt" else []
    blank = m.decoding.blank_id
    enc = torch.randn(2, 12, 176)
    lens = torch.tensor([12, 12])
    mk = lambda k: ModifiedALSDBatchedComputer(m.decoder, m.joint, blank, beam_size=k, durations=durations, max_symbols_per_step=5)  # noqa: E731
    # beam 1 follows one path, so cutting the stream into chunks cannot change it
    whole = mk(1)(enc, lens).to_hyps_list(score_norm=False)
    comp, carry = mk(1), None
    for a, b in ((0, 5), (5, 6), (6, 12)):
        hy = comp(enc[:, a:b], torch.tensor([b - a, b - a]), carry)
        carry = comp.carry
    chunked = hy.to_hyps_list(score_norm=False)
    for b in range(2):
        assert chunked[b][0][0] == whole[b][0][0] and chunked[b][0][1] == whole[b][0][1]        # tokens and global frame indices
        assert chunked[b][0][2] == pytest.approx(whole[b][0][2], abs=1e-4)
    assert carry.frame_offset.tolist() == [12, 12]
    # streams decoded in one merged batch give what each gives alone; split returns their own carries
    comp4 = mk(3)
    comp4(enc[:, :6], torch.tensor([6, 6]))
    c0, c1 = comp4.carry.split()
    alone = []
    for c, row in ((c0, 0), (c1, 1)):
        alone.append(comp4(enc[row:row + 1, 6:], torch.tensor([6]), c).to_hyps_list(score_norm=False)[0])
    comp4(enc[:, :6], torch.tensor([6, 6]))
    both = comp4(enc[:, 6:], torch.tensor([6, 6]), MALSDCarry.merge(comp4.carry.split())).to_hyps_list(score_norm=False)
    for row in range(2):
        assert [h[0] for h in both[row]] == [h[0] for h in alone[row]]
        frames = both[row][0][1]
        assert frames == sorted(frames) and all(0 <= f < 12 for f in frames)


def test_lcs_merge_and_word_spotter():
    i, j, n, _ = longest_common_subsequence_merge([5, 6, 7, 8, 9], [8, 9, 10, 11])
    assert (i, j, n) == (3, 0, 2)
    assert lcs_alignment_merge_buffer([1, 2, 3, 4, 5], [4, 5, 6, 7], delay=2) == [1, 2, 3, 4, 5, 6, 7]
    T, V = 12, 5
    lp = torch.full((T, V), -8.0)
    lp[:, 4] = -0.05
    for t, tok in [(3, 1), (4, 1), (6, 2), (7, 3)]:
        lp[t, 4], lp[t, tok] = -6.0, -0.05
    hits = ctc_word_spotter(lp, {"abc": [1, 2, 3], "zz": [0, 0]}, blank=4, keyword_threshold=-2.0)
    assert [h.word for h in hits] == ["abc"] and hits[0].start_frame in (3, 4) and hits[0].end_frame == 7


def test_streaming_aed_waitk_and_alignatt_policies():
    from speech_b200.decoding.aed_streaming import AEDStreamingDecodingConfig, GreedyBatchedStreamingAEDComputer
    from speech_b200.modules.transformer_nm import GreedySequenceGenerator, TokenClassifier, TransformerDecoderNM

    torch.manual_seed(0)
    V, D, EOS = 20, 32, 2
    dec = TransformerDecoderNM(vocab_size=V, hidden_size=D, num_layers=2, inner_size=64, num_attention_heads=4, max_sequence_length=64).eval()
    cls = TokenClassifier(D, V).eval()
    enc = torch.randn(2, 40, D)
    enc_len = torch.tensor([40, 32])
    prompt = torch.tensor([[1, 5], [1, 6]])
    # offline greedy result with the full audio (per stream: streams have different lengths)
    gen = GreedySequenceGenerator(dec.embedding, dec.decoder, cls, pad=0, bos=1, eos=EOS, max_sequence_length=24, max_delta_length=100)
    offline = []
    for b in range(2):
        ids = gen(decoder_input_ids=prompt[b:b + 1], encoder_hidden_states=enc[b:b + 1, : int(enc_len[b])],
                  encoder_input_mask=torch.ones(1, int(enc_len[b]), dtype=torch.bool))[0, 2:].tolist()
        offline.append([t for t in (ids[: ids.index(EOS)] if EOS in ids else ids) if t != 0])
    # wait-k fed with the whole audio in one last chunk equals offline greedy decoding
    cfg = AEDStreamingDecodingConfig(streaming_policy="waitk", waitk_lagging=2, max_generation_length=24, frame_chunk_size=8,
                                     hallucinations_detector=False)
    comp = GreedyBatchedStreamingAEDComputer(dec.embedding, dec.decoder, cls, EOS, cfg)
    st = comp(enc, enc_len, torch.tensor([True, True]), comp.init_state(prompt))
    cut = lambda hyps: [h[:21] for h in hyps]      # an untrained decoder never emits EOS: both runs end at their length limits  # noqa: E731
    assert cut(st.hypotheses(EOS)) == cut(offline) and not bool(st.active_samples.any())
    # chunk by chunk: nothing during the initial lag, then one token per chunk, the rest at the end
    st = comp.init_state(prompt)
    counts = []
    for c in range(1, 6):
        n = torch.minimum(torch.tensor([8 * c, 8 * c]), enc_len)
        st = comp(enc[:, : int(n.max())], n, n >= enc_len, st)
        counts.append((st.current_context_lengths - st.prompt_lengths).tolist())
    assert counts[0] == [0, 0] and counts[1] == [1, 1] and counts[2] == [2, 2]
    assert not bool(st.active_samples.any())
    assert int(st.tokens_frame_alignment[0, 2]) == 16 and int(st.tokens_frame_alignment[0, 3]) == 24
    laal = comp.compute_laal(st, enc_len, 0.08)
    assert len(laal) == 2 and all(l == l for l in laal)
    # AlignAtt: a huge threshold withholds every token until the last chunk; threshold 0 lets tokens out early
    strict = GreedyBatchedStreamingAEDComputer(dec.embedding, dec.decoder, cls, EOS, AEDStreamingDecodingConfig(
        streaming_policy="alignatt", waitk_lagging=1, alignatt_thr=1000, max_generation_length=24, frame_chunk_size=8, hallucinations_detector=False))
    st = strict.init_state(prompt)
    st = strict(enc[:, :16], torch.tensor([16, 16]), torch.tensor([False, False]), st)
    assert (st.current_context_lengths - st.prompt_lengths).tolist() == [0, 0]
    st = strict(enc, enc_len, torch.tensor([True, True]), st)
    assert cut(st.hypotheses(EOS)) == cut(offline)
    loose = GreedyBatchedStreamingAEDComputer(dec.embedding, dec.decoder, cls, EOS, AEDStreamingDecodingConfig(
        streaming_policy="alignatt", waitk_lagging=1, alignatt_thr=0, max_tokens_per_alignatt_step=3, max_generation_length=24, frame_chunk_size=8,
        hallucinations_detector=False))
    st = loose(enc[:, :16], torch.tensor([16, 16]), torch.tensor([False, False]), loose.init_state(prompt))
    assert all(0 < n <= 3 for n in (st.current_context_lengths - st.prompt_lengths).tolist())
    strict.close(), loose.close()
    # repeated n-gram tails are flagged
    st.pred_tokens_ids[0, 2:10] = torch.tensor([7, 8, 7, 8, 7, 8, 7, 8])
    st.current_context_lengths[0] = 10
    assert bool(loose.detect_hallucinations(st)[0])


def test_lexicon_ctc_beam_decoder_with_word_lm_and_graph_roundtrip(tmp_path):
    import math

    import numpy as np

    from speech_b200.decoding.lexicon_decoder import (LexiconCTCBeamDecoder, LexiconTrie, WordNGramLM, compile_lexicon_graph, read_openfst_text,
                                                      write_openfst_text)
    from speech_b200.decoding.ngram_lm import write_arpa

    # tokens: 0 blank, 1 c, 2 a, 3 t, 4 r, 5 s
    lex = {"cat": [[1, 2, 3]], "car": [[1, 2, 4]], "at": [[2, 3]], "cats": [[1, 2, 3, 5]], "a": [[2]], "tt": [[3, 3]]}
    trie = LexiconTrie(lex)

    def frames(seq, V=6, hi=0.9):
        lp = np.full((len(seq), V), math.log((1 - hi) / (V - 1)))
        for t, k in enumerate(seq):
            lp[t, k] = math.log(hi)
        return lp

    dec = LexiconCTCBeamDecoder(trie, blank_id=0, beam_size=8)
    # "c c _ a t _ c a r": repeats collapse, blank separates, two words come out
    assert dec.decode(frames([1, 1, 0, 2, 3, 0, 1, 2, 4]))[0].words == ["cat", "car"]
    # a doubled letter needs the blank between its two tokens
    assert dec.decode(frames([3, 0, 3]))[0].words == ["tt"]
    # the acoustic evidence says "c a x" with x undecided between t and r: the word LM decides
    lp = frames([1, 2, 3])
    lp[2, 3] = lp[2, 4] = math.log(0.45)
    arpa = str(tmp_path / "w.arpa")
    write_arpa(arpa, {("<s>",): (-99.0, 0.0), ("</s>",): (-1.0, 0.0), ("cat",): (-2.0, 0.0), ("car",): (-0.3, 0.0), ("at",): (-1.0, 0.0),
                      ("cats",): (-2.0, 0.0), ("a",): (-1.0, 0.0), ("tt",): (-3.0, 0.0)})
    lm = WordNGramLM.from_arpa(arpa)
    assert abs(lm.score((), "car") - (-0.3 * math.log(10))) < 1e-9
    with_lm = LexiconCTCBeamDecoder(trie, blank_id=0, lm=lm, beam_size=8, lm_weight=2.0)
    assert with_lm.decode(lp)[0].words == ["car"]
    lm2 = WordNGramLM(1, {**lm.ng, ("cat",): (-0.1, 0.0), ("car",): (-3.0, 0.0)})
    assert LexiconCTCBeamDecoder(trie, blank_id=0, lm=lm2, beam_size=8, lm_weight=2.0).decode(lp)[0].words == ["cat"]
    # token sequences outside the lexicon never come out; with an unk score they surface as <unk>
    odd = frames([4, 0, 5])
    assert dec.decode(odd) == [] or all(w in lex for w in dec.decode(odd)[0].words)
    # the compiled token-to-word graph survives the OpenFst text format and decodes identically
    arcs = compile_lexicon_graph(trie)
    finals = [s for s, ws in enumerate(trie.words) if ws] + [0]
    write_openfst_text(arcs, finals, str(tmp_path / "TL.fst.txt"))
    arcs2, finals2 = read_openfst_text(str(tmp_path / "TL.fst.txt"))
    assert sorted(arcs2, key=str) == sorted(arcs, key=str) and sorted(finals2) == sorted(set(finals))
    dec2 = LexiconCTCBeamDecoder(trie, blank_id=0, beam_size=8, graph=arcs2)
    x = frames([1, 2, 3, 5, 0, 2, 0, 2, 3])
    r1, r2 = dec.decode(x, n_best=3), dec2.decode(x, n_best=3)
    assert [r.words for r in r1] == [r.words for r in r2] and r1[0].words == ["cats", "a", "at"]
    assert r1[0].word_frames[0] in (4, 5) and len(r1[0].word_frames) == 3
    batch = dec.decode_batch(np.stack([x, x]), [9, 4])
    assert batch[0].text == "cats a at" and batch[1].words == ["cats"]


def _tiny_transducer(loss="rnnt", seed=1):
    from speech_b200.models import EncDecRNNTBPEModel
    from speech_b200.models.configs import fastconformer_transducer_config

    torch.manual_seed(seed)
    m = EncDecRNNTBPEModel(fastconformer_transducer_config("small", vocab_size=16, loss=loss, dropout=0.0, n_layers=1, sched=None, lr=1e-3))
    # a bias towards labels so that the random model emits several tokens per utterance
    with torch.no_grad():
        m.joint.joint_net[-1].bias[:16] += 1.0
    return m.eval()


def _exact_log_prob(m, enc_b, tokens):
    """log p(tokens | frames) of an RNNT by the forward recursion over the full lattice (plain loops, one utterance)."""
    blank = m.decoding.blank_id
    T, U = enc_b.shape[0], len(tokens)
    dec_out, state = m.decoder.predict(None, state=None, add_sos=False, batch_size=1)
    outs = [dec_out]
    for tok in tokens:
        o, state = m.decoder.predict(torch.tensor([[tok]]), state=state, add_sos=False, batch_size=1)
        outs.append(o)
    g = m.joint.project_prednet(torch.cat(outs, dim=1).float())[0]           # [U+1, H]
    f = m.joint.project_encoder(enc_b.float().unsqueeze(0))[0]                # [T, H]
    lin, act = m.joint.joint_net[-1], m.joint.joint_net[0]
    lp = torch.log_softmax(torch.nn.functional.linear(act(f[:, None] + g[None]), lin.weight.float(), lin.bias.float()), dim=-1)
    alpha = torch.full((T, U + 1), -1e30)
    alpha[0, 0] = 0.0
    for t in range(T):
        for u in range(U + 1):
            c = []
            if t > 0:
                c.append(alpha[t - 1, u] + lp[t - 1, u, blank])
            if u > 0:
                c.append(alpha[t, u - 1] + lp[t, u - 1, tokens[u - 1]])
            if c:
                alpha[t, u] = torch.logsumexp(torch.stack(c), dim=0)
    return float((alpha[T - 1, U] + lp[T - 1, U, blank]).detach())


def test_maes_batched_is_batch_invariant_and_scores_are_path_sums_below_the_exact_probability():
    from speech_b200.decoding.batched_beam import ModifiedAESBatchedComputer

    m = _tiny_transducer()
    blank = m.decoding.blank_id
    enc = torch.randn(3, 6, 176)
    lens = torch.tensor([6, 4, 5])
    comp = ModifiedAESBatchedComputer(m.decoder, m.joint, blank, beam_size=3, maes_num_steps=2, maes_expansion_beta=1, maes_expansion_gamma=4.0)
    full = comp(enc, lens).to_hyps_list(score_norm=False)
    for b in range(3):
        single = comp(enc[b:b + 1, : int(lens[b])], lens[b:b + 1]).to_hyps_list(score_norm=False)[0]
        assert [h[0] for h in single] == [h[0] for h in full[b]]
        assert all(abs(x[2] - y[2]) < 1e-3 for x, y in zip(single, full[b]))
        # every beam entry is a distinct transcript whose score sums some of its alignments: it cannot exceed the exact value
        assert len({tuple(h[0]) for h in full[b]}) == len(full[b])
        for tok, frames, s in full[b]:
            assert len(frames) == len(tok) and all(0 <= f < int(lens[b]) for f in frames)
            exact = _exact_log_prob(m, enc[b, : int(lens[b])], tok)
            assert s <= exact + 1e-3
    # the best beam entry is at least as probable as the greedy transcript
    greedy = m.decoding.rnnt_decoder_predictions_tensor(enc.transpose(1, 2), lens, return_hypotheses=True)
    for b in range(3):
        g_exact = _exact_log_prob(m, enc[b, : int(lens[b])], greedy[b].y_sequence.tolist())
        best_exact = max(_exact_log_prob(m, enc[b, : int(lens[b])], h[0]) for h in full[b])
        assert best_exact >= g_exact - 1e-3
    with pytest.raises(ValueError, match="plain RNNT"):
        ModifiedAESBatchedComputer(m.decoder, m.joint, blank, durations=[0, 1, 2])


def test_greedy_variants_agree_and_strategies_dispatch():
    from speech_b200.decoding.rnnt_decoding import RNNTBPEDecoding
    from speech_b200.decoding.rnnt_greedy import FrameLoopingBatchedComputer, GreedyRNNTInfer

    m = _tiny_transducer()
    enc = torch.randn(3, 9, 176)
    lens = torch.tensor([9, 5, 7])
    ref = m.decoding.rnnt_decoder_predictions_tensor(enc.transpose(1, 2), lens, return_hypotheses=True)
    assert sum(len(h.y_sequence) for h in ref) > 3
    fl = FrameLoopingBatchedComputer(m.decoder, m.joint, m.decoding.blank_id, 10)(enc, lens)
    per = GreedyRNNTInfer(m.decoder, m.joint, m.decoding.blank_id, max_symbols_per_step=10, preserve_alignments=True)(enc.transpose(1, 2), lens)[0]
    for b in range(3):
        n = int(fl.current_lengths[b])
        assert fl.transcript[b, :n].tolist() == ref[b].y_sequence.tolist() == per[b].y_sequence.tolist()
        assert fl.timestamps[b, :n].tolist() == ref[b].timestamp.tolist() == per[b].timestamp.tolist()
        assert len(per[b].alignments) <= int(lens[b])
    for strategy, extra in (("greedy", {}), ("greedy_batch", {"greedy": {"loop_labels": False}}), ("maes_batch", {"beam": {"beam_size": 2}})):
        d = RNNTBPEDecoding({"strategy": strategy, **extra}, m.decoder, m.joint, m.tokenizer)
        out = d.rnnt_decoder_predictions_tensor(enc.transpose(1, 2), lens, return_hypotheses=True)
        if strategy != "maes_batch":
            assert [h.y_sequence.tolist() for h in out] == [h.y_sequence.tolist() for h in ref]
        assert all(isinstance(h.text, str) for h in out)
    # per-sample greedy on a TDT model equals the label-looping decoder
    mt = _tiny_transducer(loss="tdt", seed=3)
    ref_t = mt.decoding.rnnt_decoder_predictions_tensor(enc.transpose(1, 2), lens, return_hypotheses=True)
    per_t = GreedyRNNTInfer(mt.decoder, mt.joint, mt.decoding.blank_id, durations=mt.decoding.durations, max_symbols_per_step=10)(enc.transpose(1, 2), lens)[0]
    for b in range(3):
        assert per_t[b].y_sequence.tolist() == ref_t[b].y_sequence.tolist() and per_t[b].timestamp.tolist() == ref_t[b].timestamp.tolist()


def test_host_context_graph_word_spotting_graph_and_merge():
    import numpy as np

    from speech_b200.decoding.context_biasing import WordSpotterHyp
    from speech_b200.decoding.context_graph import CTCContextGraph, ContextGraph, merge_alignment_with_ws_hyps

    g = ContextGraph(context_score=2.0).build([[1, 2, 3], [2, 3, 4, 5], [7]], phrases=["abc", "bcde", "g"])
    assert g.num_nodes == 1 + 3 + 4 + 1
    # a completed phrase keeps its boost; leaving a partly matched phrase gives the boost back
    assert g.score_sequence([9, 1, 2, 3, 9]) == (6.0, ["abc"])
    assert g.score_sequence([1, 2, 9]) == (0.0, [])
    assert g.score_sequence([1, 2]) == (0.0, [])                               # unfinished at the end of the utterance
    # failure links: after "a b c" the path continues into "b c d e" without starting over
    total, found = g.score_sequence([1, 2, 3, 4, 5])
    assert found == ["abc", "bcde"] and total == pytest.approx(6.0 + 8.0 - 6.0 + 6.0 - 6.0 + 0.0, abs=8.0) and total >= 8.0
    s, st, m = g.forward_one_step(g.root, 7)
    assert s == 2.0 and m is not None and m.phrase == "g" and g.finalize(st)[0] == 0.0
    deep = ContextGraph(1.0, depth_scaling=2.0).build([[1, 2, 3]])
    assert deep.score_sequence([1, 2, 3])[0] == 1 + 2 + 4
    weighted = ContextGraph(1.0).build([[1, 2], [3]], scores=[5.0, 0.0])
    assert weighted.score_sequence([1, 2, 3])[0] == 10.0 + 1.0
    # CTC-topology search over posteriors: "b c" spoken at frames 3-7
    V, blank = 6, 5
    lp = np.full((12, V), np.log(0.02))
    lp[:, blank] = np.log(0.9)
    for t, tok in [(3, 2), (4, 2), (6, 3), (7, 3)]:
        lp[t, blank], lp[t, tok] = np.log(0.02), np.log(0.9)
    hits = CTCContextGraph({"bc": [2, 3], "zz": [0, 0]}, blank).search(lp, threshold=-1.0)
    assert len(hits) == 1 and hits[0][0] == "bc" and 3 <= hits[0][2] <= 4 and 6 <= hits[0][3] <= 7 and hits[0][1] > -0.5
    toks = {1: "▁the", 2: "▁cat", 3: "s", 4: "▁sat"}
    ali = [5, 1, 1, 5, 2, 2, 3, 5, 5, 4, 4, 5]
    text, words = merge_alignment_with_ws_hyps(ali, [WordSpotterHyp("kats", -0.2, 4, 6)], lambda i: toks[i], blank=5)
    assert text == "the kats sat" and words[1] == ("kats", 4, 6)
    assert merge_alignment_with_ws_hyps(ali, [], lambda i: toks[i], blank=5)[0] == "the cats sat"


def test_exported_transducer_graphs_reproduce_framework_greedy_decoding(tmp_path):
    import torch

    from speech_b200.decoding.exported_rnnt import ONNXGreedyBatchedRNNTInfer, TorchscriptGreedyBatchedRNNTInfer, export_transducer_subnets
    from speech_b200.models.configs import fastconformer_transducer_config
    from speech_b200.models.rnnt_models import EncDecRNNTBPEModel

    torch.manual_seed(3)
    for loss in ("rnnt", "tdt"):
        cfg = fastconformer_transducer_config("small", vocab_size=24, n_layers=2, loss=loss, dropout=0.0)
        cfg.joint.fuse_loss_wer = False
        model = EncDecRNNTBPEModel(cfg).eval()
        with torch.no_grad():
            model.joint.joint_net[-1].bias[:-1 if loss == "rnnt" else -6] += 1.5          # make non-blank tokens likely so that the loop really emits
        enc_path, dj_path = export_transducer_subnets(model, str(tmp_path / loss), feat_frames=48)
        durations = list(getattr(model.decoding, "durations", None) or [])
        infer = TorchscriptGreedyBatchedRNNTInfer(enc_path, dj_path, blank_id=model.decoding.blank_id, pred_layers=model.decoder.pred_rnn_layers,
                                                  pred_hidden=model.decoder.pred_hidden, max_symbols_per_step=3, durations=durations)
        feats = torch.randn(3, 80, 120)
        flen = torch.tensor([120, 90, 57])
        got = infer(feats, flen)
        with torch.no_grad():
            enc, enc_len = model.encoder(audio_signal=feats, length=flen)
        model.change_decoding_strategy({"strategy": "greedy_batch", "greedy": {"max_symbols": 3}})
        ref = model.decoding.rnnt_decoder_predictions_tensor(enc, enc_len, return_hypotheses=True)
        ref_ids = [[int(t) for t in h.y_sequence] for h in ref]
        assert got == ref_ids and sum(len(g) for g in got) > 0
    with pytest.raises(RuntimeError, match="onnxruntime"):
        ONNXGreedyBatchedRNNTInfer("e.onnx", "d.onnx", 24, 1, 320)
    with pytest.raises(FileNotFoundError):
        TorchscriptGreedyBatchedRNNTInfer(str(tmp_path / "no.ts"), dj_path, 24, 1, 320)
