"""Streaming inference on CPU: slot allocator, continuous batching, cache-aware and buffered pipelines.

The cache-aware check follows the reference's own oracle: chunk-by-chunk decoding with caches must give the same tokens as
the offline encoder run with the same limited-context mask."""
import numpy as np
import pytest
import torch

from speech_b200.core.config import open_dict
from speech_b200.inference.context_manager import CacheAwareContextManager
from speech_b200.inference.framing import ContinuousBatchedRequestStreamer, RequestType
from speech_b200.inference.pipelines import PipelineBuilder
from speech_b200.inference.state import GreedyEndpointing, StreamingState, TokenTextAssembler
from speech_b200.models import EncDecCTCModelBPE, EncDecRNNTBPEModel
from speech_b200.models.configs import fastconformer_ctc_config, fastconformer_transducer_config


def _streaming_overrides(cfg):
    with open_dict(cfg):
        cfg.preprocessor.normalize = "NA"
        cfg.preprocessor.dither = 0.0
        cfg.preprocessor.pad_to = 0
    return cfg


def _audio(n, seed):
    g = np.random.default_rng(seed)
    return (g.standard_normal(n) * 0.1).astype(np.float32)


def test_streamer_keeps_batch_full_and_orders_chunks():
    s = ContinuousBatchedRequestStreamer(n_frames_per_stream=1000, batch_size=2, sample_rate=16000)
    s.set_audio_filepaths([_audio(2500, 0), _audio(900, 1), _audio(1800, 2)])
    steps = [[(f.stream_id, f.is_first, f.is_last, f.valid_size) for f in batch] for batch in s]
    assert steps[0] == [(0, True, False, 1000), (1, True, True, 900)]
    assert steps[1] == [(0, False, False, 1000), (2, True, False, 1000)]   # stream 2 joined as soon as stream 1 ended
    assert steps[2] == [(0, False, True, 500), (2, False, True, 800)]
    assert len(steps) == 3


class _FakeEncoder:
    def get_initial_cache_state(self, batch_size=1):
        return torch.zeros(2, batch_size, 4, 3), torch.zeros(2, batch_size, 3, 2), torch.zeros(batch_size, dtype=torch.long)


def test_context_manager_slots_gather_scatter_and_reuse():
    cm = CacheAwareContextManager(_FakeEncoder(), num_slots=3)
    ctx, mp = cm.get_context([10, 11])
    assert ctx.cache_last_channel.shape == (2, 2, 4, 3) and cm.num_free_slots() == 1
    ctx.cache_last_channel = torch.ones(2, 2, 4, 3) * torch.tensor([1.0, 2.0]).view(1, 2, 1, 1)
    ctx.cache_last_time = torch.ones(2, 2, 3, 2)
    ctx.cache_last_channel_len = torch.tensor([4, 2])
    cm.update_cache([10, 11], ctx, mp)
    again, _ = cm.get_context([11, 10])
    assert float(again.cache_last_channel[0, 0, 0, 0]) == 2.0 and again.cache_last_channel_len.tolist() == [2, 4]
    cm.reset_slots([10, 11], [True, False])
    assert cm.num_free_slots() == 2
    fresh, _ = cm.get_context([12])
    assert float(fresh.cache_last_channel.abs().sum()) == 0.0       # the freed slot was zeroed
    with pytest.raises(RuntimeError):
        cm.get_context([13, 14, 15])


def test_endpointing_and_word_assembly():
    toks = {1: "▁he", 2: "llo", 3: "▁wor", 4: "ld"}
    asm = TokenTextAssembler(lambda ids: [toks[i] for i in ids],
                             lambda ids: "".join(toks[i] for i in ids).replace("▁", " ").strip(), seconds_per_frame=0.08)
    ws = asm.words([1, 2, 3, 4], [0, 2, 10, 11], [0.9, 0.7, 1.0, 0.5])
    assert [w.text for w in ws] == ["hello", "world"]
    assert ws[0].start == 0.0 and abs(ws[0].end - 0.24) < 1e-9 and abs(ws[0].conf - 0.8) < 1e-9
    st = StreamingState(0)
    ep = GreedyEndpointing(ms_per_frame=80.0, stop_history_eou_ms=400)
    st.append_tokens([1, 2], [0, 1])
    st.advance(4)
    assert not ep.detect_eou(st)
    st.advance(4)                      # 6 silent frames >= 5
    assert ep.detect_eou(st) and ep.detect_eou(StreamingState(1), is_last=True)


@pytest.mark.parametrize("kind", ["ctc", "rnnt"])
def test_cache_aware_pipeline_matches_offline_limited_context(kind):
    torch.manual_seed(0)
    enc_over = dict(n_layers=2, causal=True, att_context_size=[8, 1], att_context_style="chunked_limited",
                    conv_norm_type="layer_norm")
    if kind == "ctc":
        model = EncDecCTCModelBPE(_streaming_overrides(fastconformer_ctc_config("small", vocab_size=32, **enc_over)))
    else:
        model = EncDecRNNTBPEModel(_streaming_overrides(fastconformer_transducer_config(
            "small", vocab_size=32, loss="rnnt", dropout=0.0, sched=None, lr=1e-3, **enc_over)))
    model.eval()
    audios = [_audio(16000 * 2 + 320, 1), _audio(16000 + 4000, 2), _audio(16000 * 3, 3)]
    pipe = PipelineBuilder.build_pipeline({"pipeline_type": "cache_aware",
                                           "streaming": {"batch_size": 2, "num_slots": 4},
                                           "endpointing": {"stop_history_eou": 100000}}, asr_model=model)
    out = pipe.run(audios)
    assert sorted(out) == [0, 1, 2]
    offline = model.transcribe(audios, batch_size=1)
    off_text = [h.text if hasattr(h, "text") else h for h in offline]
    # same limited-context encoder offline and online, offline-exact feature frames: identical token streams
    for i in range(3):
        assert out[i].text.split() == off_text[i].split(), i
    assert pipe.rtfx() > 0


def test_cache_aware_rnnt_pipeline_with_a_beam_carried_between_chunks():
    torch.manual_seed(0)
    enc_over = dict(n_layers=2, causal=True, att_context_size=[8, 1], att_context_style="chunked_limited", conv_norm_type="layer_norm")
    model = EncDecRNNTBPEModel(_streaming_overrides(fastconformer_transducer_config(
        "small", vocab_size=32, loss="rnnt", dropout=0.0, sched=None, lr=1e-3, **enc_over))).eval()
    audios = [_audio(16000 * 2 + 320, 1), _audio(16000 + 4000, 2), _audio(16000 * 3, 3)]

    def run(beam):
        pipe = PipelineBuilder.build_pipeline({"pipeline_type": "cache_aware", "streaming": {"batch_size": 2, "num_slots": 4},
                                               "endpointing": {"stop_history_eou": 100000},
                                               "asr": {"decoding": {"strategy": "malsd_batch", "beam": {"beam_size": beam}}}}, asr_model=model)
        assert pipe.malsd is not None and pipe.malsd.K == beam
        return pipe.run(audios)

    greedy = PipelineBuilder.build_pipeline({"pipeline_type": "cache_aware", "streaming": {"batch_size": 2, "num_slots": 4},
                                             "endpointing": {"stop_history_eou": 100000}}, asr_model=model).run(audios)
    one, four = run(1), run(4)
    for i in range(3):
        assert one[i].text == greedy[i].text, i                # a beam of one is the greedy path, chunk boundaries included
        assert isinstance(four[i].text, str)
        times = [w.start for w in four[i].words]
        assert times == sorted(times)


def test_cache_aware_pipeline_full_batch_in_slot_order_skips_the_gather():
    """A batch that holds every slot in order reads the resident caches directly; the tokens equal the offline ones."""
    torch.manual_seed(0)
    model = EncDecCTCModelBPE(_streaming_overrides(fastconformer_ctc_config(
        "small", vocab_size=32, n_layers=2, causal=True, att_context_size=[8, 1], att_context_style="chunked_limited",
        conv_norm_type="layer_norm")))
    model.eval()
    audios = [_audio(16000 * 2, 1), _audio(16000 * 2, 2), _audio(16000 * 2, 3)]
    pipe = PipelineBuilder.build_pipeline({"pipeline_type": "cache_aware", "streaming": {"batch_size": 3, "num_slots": 3},
                                           "endpointing": {"stop_history_eou": 100000}}, asr_model=model)
    cm = pipe.context_manager
    seen = []
    orig = cm.get_context

    def spy(ids):
        ctx, mp = orig(ids)
        seen.append(ctx.cache_last_channel.data_ptr() == cm.cache_last_channel.data_ptr())
        return ctx, mp

    cm.get_context = spy
    out = pipe.run(audios)
    assert any(seen)                                                   # the resident tensors were handed out as they are
    off_text = [h.text if hasattr(h, "text") else h for h in model.transcribe(audios, batch_size=1)]
    for i in range(3):
        assert out[i].text.split() == off_text[i].split(), i


def test_buffered_ctc_pipeline_runs_and_times_words():
    torch.manual_seed(0)
    model = EncDecCTCModelBPE(_streaming_overrides(fastconformer_ctc_config("small", vocab_size=32, n_layers=1)))
    model.eval()
    pipe = PipelineBuilder.build_pipeline({"pipeline_type": "buffered",
                                           "streaming": {"batch_size": 2, "chunk_size": 0.8, "left_padding_size": 0.8,
                                                         "right_padding_size": 0.4}}, asr_model=model)
    out = pipe.run([_audio(16000 * 2, 5), _audio(12000, 6)])
    assert sorted(out) == [0, 1]
    for o in out.values():
        assert isinstance(o.text, str)
        for w in o.words:
            assert 0.0 <= w.start <= w.end


def test_inverse_text_normalisation_and_translation_hook():
    from speech_b200.inference.text_postprocess import InverseTextNormalizer, TranslationHook

    n = InverseTextNormalizer()
    assert n("i have twenty three apples and one hundred and five pears") == "i have 23 apples and 105 pears"
    assert n("it costs fifteen dollars or three point one four percent") == "it costs $15 or 3.14%"
    assert n("the twenty first of may at seven o'clock") == "the 21st of may at 7:00"
    assert n("two thousand twenty five was the third year") == "2025 was the 3rd year"
    assert n("one of them came forty-second") == "one of them came 42nd"
    assert n.normalize_list(["one hundred", "no numbers"]) == ["100", "no numbers"]
    hook = TranslationHook(lambda xs: [x.upper() for x in xs], batch_size=2)
    assert hook(["a", "b", "c"]) == ["A", "B", "C"]
    import pytest

    with pytest.raises(RuntimeError):
        TranslationHook(lambda xs: xs[:-1])(["a", "b"])


def test_voice_agent_pipeline_turns_tools_and_barge_in(tmp_path):
    import os

    import numpy as np

    from speech_b200.agents.voice_agent import (AudioRawFrame, BotInterruptionFrame, EndFrame, LLMTextFrame, ToolCallFrame, TranscriptionFrame,
                                                TTSAudioFrame, UserStoppedSpeakingFrame, build_voice_agent)

    heard = []

    def stt(chunk):                       # a stand-in recogniser: one more word per loud chunk
        if float(np.abs(chunk).mean()) > 0.05:
            heard.append("word")
        return " ".join(heard), False

    calls = []

    def llm(messages):
        calls.append([m["role"] for m in messages])
        if messages[-1]["role"] == "tool":
            return "It is 7 degrees. Bring a coat!"
        return '{"tool": "weather", "arguments": {"city": "Oslo"}}'

    def tts(text):
        return np.full(800, 0.1, np.float32), 8000

    agent = build_voice_agent(stt, llm, tts, diar_step=lambda a: np.tile(np.array([[0.1, 0.9]]), (4, 1)), log_dir=str(tmp_path),
                              system_prompt="be brief", tools={"weather": lambda city: {"city": city, "temp_c": 7}}, max_silence=0.3)
    sr = 16000
    loud, quiet = np.full(1600, 0.2, np.float32), np.zeros(1600, np.float32)
    frames = [AudioRawFrame(0.1 * i, loud, sr) for i in range(5)] + [AudioRawFrame(0.5 + 0.1 * i, quiet, sr) for i in range(4)]
    out = agent.run(frames)
    kinds = [type(f).__name__ for f in out]
    assert "UserStartedSpeakingFrame" in kinds and "UserStoppedSpeakingFrame" in kinds
    finals = [f for f in out if isinstance(f, TranscriptionFrame) and f.is_final]
    assert len(finals) == 1 and finals[0].text == "word word word word word" and finals[0].speaker == "speaker_1"
    tool = [f for f in out if isinstance(f, ToolCallFrame)]
    assert tool and tool[0].result == {"city": "Oslo", "temp_c": 7}
    reply = [f for f in out if isinstance(f, LLMTextFrame)]
    assert reply[0].text == "It is 7 degrees. Bring a coat!" and calls[0] == ["system", "user"] and calls[1][-1] == "tool"
    audio = [f for f in out if isinstance(f, TTSAudioFrame)]
    assert [a.text for a in audio] == ["It is 7 degrees.", "Bring a coat!"]           # sentence-wise synthesis
    # barge-in: the user speaks while the bot is talking
    heard.clear()
    out2 = agent.run([TTSAudioFrame(2.0, np.zeros(10, np.float32), 8000, "x")] + [AudioRawFrame(2.0 + 0.1 * i, loud, sr) for i in range(3)])
    assert any(isinstance(f, BotInterruptionFrame) for f in out2)
    agent.run([EndFrame(9.0)])
    assert os.path.exists(tmp_path / "session" / "user.wav") and os.path.exists(tmp_path / "session" / "bot.wav")
    lines = open(tmp_path / "session" / "events.jsonl").read().strip().splitlines()
    assert any('"LLMTextFrame"' in l for l in lines)


def test_chunked_aed_inference_merges_short_tail():
    from speech_b200.utils.streaming_utils import BatchedFrameASRRNNT, BatchedFrameASRTDT, FrameBatchMultiTaskAED

    class M:
        def transcribe(self, audio, batch_size=1, **kw):
            return [f"len{len(a)}" for a in audio]

    f = FrameBatchMultiTaskAED(M(), chunk_len=1.0, batch_size=2, min_tail=0.5, sample_rate=100)
    f.read_audio_file(torch.zeros(330))
    assert f.transcribe() == "len100 len100 len130" and BatchedFrameASRTDT is BatchedFrameASRRNNT


def test_buffered_salm_pipeline_merges_window_transcripts_by_overlap():
    from speech_b200.inference.pipelines import BufferedSALMPipeline, merge_by_word_overlap

    assert merge_by_word_overlap("a b c d".split(), "c d e f".split()) == "a b c d e f".split()
    assert merge_by_word_overlap([], ["x"]) == ["x"] and merge_by_word_overlap(["a"], ["b"]) == ["a", "b"]

    class _Tok:
        words = ["zero", "one", "two", "three", "four", "five", "six", "seven"]

        def ids_to_text(self, ids):
            return " ".join(self.words[i] for i in ids)

    class _FakeSALM:
        """Speaks one word per half second of audio: the word index is the absolute half-second index, recovered from the
        sample values (each stream's audio is a ramp of its half-second index)."""
        tokenizer, text_eos_id, text_pad_id, audio_locator_tag = _Tok(), 98, 99, "<|audioplaceholder|>"
        calls = []

        def generate(self, dialogs, audios, audio_lens, max_new_tokens):
            assert all("<|audioplaceholder|>" in d[0]["content"] for d in dialogs)
            self.calls.append(tuple(int(n) for n in audio_lens))
            rows = []
            for a, n in zip(audios, audio_lens):
                idx = [int(round(float(a[k * 8000 + 4000]))) for k in range(int(n) // 8000)]
                rows.append(idx + [98] + [99] * (max_new_tokens - len(idx) - 1))
            return torch.tensor(rows)

    audio = torch.cat([torch.full((8000,), float(k)) for k in range(8)]).numpy()          # 4 s, half second k holds the value k
    pipe = BufferedSALMPipeline({"streaming": {"batch_size": 2, "chunk_size": 1.0, "left_padding_size": 1.0}, "salm": {"max_new_tokens": 8}}, _FakeSALM())
    out = pipe.run([audio, audio[: 8000 * 5]])
    assert out[0].text == "zero one two three four five six seven"
    assert out[1].text == "zero one two three four"
    # the first step sees one second, later steps the two-second window
    assert pipe.salm.calls[0] == (16000, 16000) and pipe.salm.calls[1] == (32000, 32000)


def test_alignment_preserving_itn_keeps_word_times_and_merges_punctuation():
    from speech_b200.inference.state import Word
    from speech_b200.inference.text_postprocess import (AlignmentPreservingInverseNormalizer, BatchAlignmentPreservingInverseNormalizer,
                                                        merge_punctuation_and_itn)

    itn = AlignmentPreservingInverseNormalizer()
    words = "it costs twenty five dollars and the third one is fifty percent off".split()
    src, out, spans = itn.get_word_alignment(words)
    assert out == "it costs $25 and the 3rd one is 50% off".split()
    assert (2, 5, 2, 3) in spans and (7, 8, 5, 6) in spans and (10, 12, 8, 9) in spans
    assert sorted(i for a, b, _, _ in spans for i in range(a, b)) == list(range(len(words)))       # a partition of the input
    assert sorted(o for _, _, a, b in spans for o in range(a, b)) == list(range(len(out)))         # and of the output
    ws = [Word(text=w, start=0.5 * i, end=0.5 * i + 0.4, conf=0.9 if w != "five" else 0.5) for i, w in enumerate(words)]
    new = itn.apply_to_words(ws)
    price = next(w for w in new if w.text == "$25")
    assert price.start == 1.0 and price.end == pytest.approx(2.4) and price.conf == 0.5
    pnc = "It costs twenty five dollars, and the third one is fifty percent off.".split()
    assert merge_punctuation_and_itn(pnc, out, spans) == "It costs $25, and the 3rd one is 50% off.".split()
    batch = BatchAlignmentPreservingInverseNormalizer(itn, n_jobs=2)([ws, ws[:2]], [pnc, None])
    assert [w.text for w in batch[0]] == "It costs $25, and the 3rd one is 50% off.".split() and [w.text for w in batch[1]] == ["it", "costs"]


def test_llm_translator_continues_a_stable_prefix():
    from speech_b200.inference.text_postprocess import LLMTranslator, TranslationPrompt

    seen = []

    def engine(prompts):
        seen.extend(prompts)
        # a toy "model": continues the prefix with upper-cased source words it has not produced yet
        outs = []
        for p in prompts:
            src = p.split("English: ")[1].split("\n")[0].split()
            prefix = p.split("assistant\n")[1]
            done = len(prefix.split())
            outs.append((" " if prefix else "") + " ".join(w.upper() for w in src[done:]) + "<|im_end|> ignored")
        return outs

    tr = LLMTranslator(engine, waitk=2, batch_size=1)
    t1 = tr.translate(["hello my"], [""], ["en"], ["de"])
    assert t1 == ["HELLO MY"] and "Translate the following English source text to German" in seen[0] and seen[0].endswith("assistant\n")
    assert TranslationPrompt.extract("abc\ndef") == "abc"
    # the next step agrees with the previous one on "HELLO M": cut back to the word boundary
    assert tr.get_prefixes(["hello my dear"], ["HELLO MX DEAR"], ["HELLO MY"]) == ["HELLO"]
    # the translations disagree from the start while the transcript has 6 words: the prefix is forced to 6 - waitk words
    assert tr.get_prefixes(["a b c d e f"], ["U V W X Y Z"], ["K L"]) == ["U V W X"]
    assert tr.get_prefixes([""], ["HALLUCINATION"], ["HALLUCINATION"]) == [""]
    t2 = tr.translate(["hello my dear friend"], ["HELLO"], ["en"], ["de"])
    assert t2 == ["HELLO MY DEAR FRIEND"]


def test_left_chunk_right_buffer_accounting_and_chunked_inference():
    from speech_b200.utils.streaming_buffers import (AudioBatch, AudioFeatureIterator, BatchedFeatureFrameBufferer, ContextSize, FrameBatchChunkedCTC,
                                                     FrameBatchChunkedRNNT, LongestCommonSubsequenceBatchedFrameASRRNNT, SimpleAudioDataset,
                                                     StreamingBatchedAudioBuffer, StreamingFeatureBufferer, inplace_buffer_merge)

    exp = ContextSize(left=6, chunk=4, right=2)
    buf = StreamingBatchedAudioBuffer(2, exp)
    stream = torch.arange(1, 21, dtype=torch.float32)[None].repeat(2, 1)
    lens_total = torch.tensor([20, 13])                                  # the second stream is shorter
    pos, seen = 0, []
    first = True
    while pos < 20:
        n = exp.chunk + exp.right if first else exp.chunk
        n = min(n, 20 - pos)
        last = pos + n >= 20
        lens = (lens_total - pos).clamp(min=0, max=n)
        buf.add_audio_batch_(stream[:, pos:pos + n], lens, last, lens_total <= pos + n)
        c = buf.context_size
        assert buf.samples.shape[1] == c.total() <= exp.total()
        chunk = buf.samples[0, c.left: c.left + c.chunk]
        seen += chunk.tolist()
        if not last:
            assert c.chunk == exp.chunk and c.right == exp.right
        pos, first = pos + n, False
    assert seen == list(range(1, 21))                                    # every sample is the "chunk" exactly once, in order
    assert buf.context_size.left == 8 and buf.context_size.right == 0          # no look-ahead is left, so the left context may use its room
    b = buf.context_size_batch
    assert int(b.right[1]) == 0 and int(b.total()[1]) <= exp.total()
    assert inplace_buffer_merge([1, 2, 3, 4], [9, 8, 7], 2) == [1, 2, 9, 8, 7]

    torch.manual_seed(0)
    ctc = EncDecCTCModelBPE(_streaming_overrides(fastconformer_ctc_config("small", vocab_size=32, n_layers=1))).eval()
    audio = _audio(16000 * 3, 5)
    # incremental features equal whole-signal features
    sfb = StreamingFeatureBufferer(ctc, chunk_size=0.5, buffer_size=4.0)
    for k in range(0, 48000, 8000):
        out = sfb.append(audio[k:k + 8000])
    assert sfb.frames_seen == 299                                        # the newest half window waits for more samples
    out = sfb.flush()
    whole, _ = ctc.preprocessor(input_signal=torch.tensor(audio)[None], length=torch.tensor([48000]))
    assert sfb.frames_seen == whole.shape[2] == 301 and torch.allclose(out[:, -301:], whole[0], atol=1e-4)
    it = AudioFeatureIterator(audio, 1.0, ctc.preprocessor)
    frames = list(it)
    assert len(frames) == 3 and frames[0].shape == (80, 100)              # 300 valid frames
    bb = BatchedFeatureFrameBufferer(ctc, frame_len=1.0, total_buffer=2.0)
    bb.set_frame_reader(AudioFeatureIterator(audio, 1.0, ctc.preprocessor), 0)
    bb.set_frame_reader(AudioFeatureIterator(audio[:16000], 1.0, ctc.preprocessor), 1)
    steps = []
    while True:
        bufs, ids = bb.get_buffers_batch()
        if not bufs:
            break
        steps.append(ids)
        assert all(x.shape == (80, 200) for x in bufs)
    assert steps[0] == [0, 1] and steps[-1] == [0]
    chunked = FrameBatchChunkedCTC(ctc, frame_len=1.0, batch_size=2)
    chunked.read_audio_file(audio)
    assert isinstance(chunked.transcribe(), str) and len(chunked.all_preds) == 3
    rnnt = EncDecRNNTBPEModel(_streaming_overrides(fastconformer_transducer_config("small", vocab_size=32, loss="rnnt", dropout=0.0, sched=None, lr=1e-3,
                                                                                   n_layers=1))).eval()
    for cls, kw in ((FrameBatchChunkedRNNT, dict(frame_len=1.0)), (LongestCommonSubsequenceBatchedFrameASRRNNT, dict(frame_len=0.8, total_buffer=2.4))):
        d = cls(rnnt, batch_size=2, **kw)
        d.read_audio_file(audio)
        assert isinstance(d.transcribe(), str)
    ds = SimpleAudioDataset([audio, audio[:1000]])
    batch = AudioBatch.collate_fn([ds[0], ds[1]])
    assert batch.audio_signals.shape == (2, 48000) and batch.audio_signal_lengths.tolist() == [48000, 1000] and batch.ids.tolist() == [0, 1]


def test_streaming_transducer_inference_with_left_and_right_context():
    from speech_b200.utils.streaming_buffers import streaming_transcribe_rnnt

    torch.manual_seed(0)
    rnnt = EncDecRNNTBPEModel(_streaming_overrides(fastconformer_transducer_config("small", vocab_size=32, loss="rnnt", dropout=0.0, sched=None, lr=1e-3,
                                                                                   n_layers=1))).eval()
    audio = torch.tensor(np.stack([_audio(32000, 1), _audio(32000, 2)]))
    lens = torch.tensor([32000, 20000])
    audio[1, 20000:] = 0
    offline = rnnt.transcribe([audio[0].numpy(), audio[1, :20000].numpy()], batch_size=2, return_hypotheses=True)
    # one chunk that holds everything is the offline pass
    one = streaming_transcribe_rnnt(rnnt, audio[:1], lens[:1], chunk_secs=4.0, left_context_secs=0.0, right_context_secs=0.0)
    assert [int(t) for t in one[0].y_sequence] == [int(t) for t in offline[0].y_sequence]
    hyps = streaming_transcribe_rnnt(rnnt, audio, lens, chunk_secs=0.48, left_context_secs=0.96, right_context_secs=0.24)
    assert len(hyps) == 2 and all(h is not None for h in hyps)
    ts = [int(t) for t in (hyps[0].timestamp.tolist() if torch.is_tensor(hyps[0].timestamp) else hyps[0].timestamp)]
    assert ts == sorted(ts)


def test_inference_option_enums_parse_config_strings():
    from speech_b200.inference.enums import ASRDecodingType, FeatureBufferPaddingMode, MergingStrategy, PipelineType, RequestType

    assert PipelineType.from_str("Cache_Aware") is PipelineType.CACHE_AWARE and MergingStrategy.from_str("lcsubstr") is MergingStrategy.LCSUBSTR
    assert FeatureBufferPaddingMode.from_str("left") is FeatureBufferPaddingMode.LEFT and RequestType.FRAME is not RequestType.FEATURE_BUFFER
    with pytest.raises(ValueError, match="ctc"):
        ASRDecodingType.from_str("transducer")
