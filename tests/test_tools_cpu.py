"""Command-line helpers: duration bins, tarred conversion, n-gram LM training, forced alignment, checkpoint averaging,
tokenizer building, batch-size search."""
import json
import math
import os

import numpy as np
import pytest
import torch

from speech_b200.data import tools
from speech_b200.data.audio_to_text import read_manifest, save_wav
from speech_b200.decoding.forced_aligner import viterbi_ctc_alignment
from speech_b200.decoding.ngram_lm import NGramGPULanguageModel, write_arpa
from speech_b200.decoding.train_ngram_lm import train_ngram
from speech_b200.utils.checkpoint_averaging import average_state_dicts
from speech_b200.utils.oomptimizer import find_max_batch


def _corpus(tmp_path, n=10):
    g = np.random.default_rng(0)
    man = str(tmp_path / "m.json")
    with open(man, "w") as f:
        for i in range(n):
            p = str(tmp_path / f"a{i}.wav")
            save_wav(p, (0.1 * g.standard_normal(1600 * (i + 1))).astype(np.float32))
            f.write(json.dumps({"audio_filepath": p, "duration": 0.1 * (i + 1), "text": "hello world " * (1 + i % 3)}) + "\n")
    return man


def test_duration_bins_weights_and_tarred_conversion(tmp_path):
    man = _corpus(tmp_path)
    bins = tools.estimate_duration_bins([man], 3)
    assert len(bins) == 2 and bins == sorted(bins) and 0.1 < bins[0] < bins[1] < 1.0
    w = tools.estimate_data_weights({"a": man, "b": man}, temperature=0.5)
    assert abs(w["a"] - 0.5) < 1e-9
    meta = tools.convert_to_tarred(man, str(tmp_path / "tar"), num_shards=3, seed=1)
    assert meta["num_samples_per_shard"] == 3 and meta["dropped"] == 1
    from speech_b200.data.cuts import read_nemo_tarred

    cuts = list(read_nemo_tarred(str(tmp_path / "tar" / "tarred_audio_manifest.json"), str(tmp_path / "tar" / "audio__OP_0..2_CL_.tar")))
    assert len(cuts) == 9 and all(abs(len(c.audio) / 16000 - c.duration) < 1e-3 for c in cuts)
    tools.main(["filter-manifest", man, str(tmp_path / "f.json"), "--max-duration", "0.5"])
    assert len(read_manifest(str(tmp_path / "f.json"))) == 5


def test_ngram_training_normalises_and_prefers_seen_sequences(tmp_path):
    sents = [[0, 1, 2], [0, 1, 3], [0, 1, 2], [4, 1, 2]] * 5
    grams = train_ngram(sents, order=3, vocab_size=5)
    arpa = str(tmp_path / "lm.arpa")
    write_arpa(arpa, grams)
    lm = NGramGPULanguageModel.from_arpa(arpa, vocab_size=5)
    st = lm.get_init_states(1, bos=True)
    sc, nx = lm.advance(st)
    total = float(torch.logsumexp(torch.cat([sc[0], lm.get_final(st)]), 0))
    assert abs(total) < 0.05                                    # p(. | <s>) sums to ~1 over tokens + </s> (unk mass aside)
    assert lm.score_sentence([0, 1, 2]) > lm.score_sentence([2, 1, 0]) + 2.0
    st = nx[:, 0]
    sc, nx = lm.advance(st)
    assert int(sc[0].argmax()) == 1


def test_viterbi_alignment_finds_the_planted_path():
    T, V, blank = 12, 5, 4
    lp = torch.full((T, V), -6.0)
    lp[:, blank] = -0.5
    for t, tok in [(2, 1), (3, 1), (6, 2), (9, 1)]:
        lp[t, tok], lp[t, blank] = -0.05, -5.0
    spans = viterbi_ctc_alignment(lp, [1, 2, 1], blank)
    assert [(a, b) for a, b, _ in spans] == [(2, 3), (6, 6), (9, 9)]
    assert viterbi_ctc_alignment(lp, [], blank) == []
    with pytest.raises(ValueError):
        viterbi_ctc_alignment(lp[:2], [1, 2, 1], blank)


def test_checkpoint_averaging_and_batch_search():
    a = {"w": torch.tensor([1.0, 3.0]), "n": torch.tensor(5)}
    b = {"w": torch.tensor([3.0, 5.0]), "n": torch.tensor(9)}
    avg = average_state_dicts([a, b])
    assert avg["w"].tolist() == [2.0, 4.0] and int(avg["n"]) == 5
    calls = []
    assert find_max_batch(lambda n: (calls.append(n) or n <= 37), start=1, limit=4096) in range(35, 38)
    assert find_max_batch(lambda n: False) == 0 and find_max_batch(lambda n: True, limit=64) == 64


def test_tokenizer_builder(tmp_path):
    from speech_b200.tokenizers import SentencePieceTokenizer, WordPieceVocabTokenizer
    from speech_b200.tokenizers.process_asr_text_tokenizer import main

    man = _corpus(tmp_path, 6)
    main(["--manifest", man, "--data_root", str(tmp_path / "tok"), "--vocab_size", "20", "--tokenizer", "spe", "--spe_type", "bpe"])
    tok = SentencePieceTokenizer(str(tmp_path / "tok" / "tokenizer_spe_bpe_v20" / "tokenizer.model"))
    assert tok.ids_to_text(tok.text_to_ids("hello world")) == "hello world"
    main(["--manifest", man, "--data_root", str(tmp_path / "tok"), "--vocab_size", "30", "--tokenizer", "wpe"])
    wp = WordPieceVocabTokenizer(str(tmp_path / "tok" / "tokenizer_wpe_v30" / "vocab.txt"))
    assert wp.ids_to_text(wp.text_to_ids("hello world")) == "hello world"


def test_voice_agent_websocket_transport_and_server_app():
    """The transport re-frames client audio, forwards pipeline events as JSON and the bot's speech as PCM; the example server's app
    answers a whole conversation through a fake websocket (no network)."""
    import asyncio
    import importlib.util
    import json
    import os

    import numpy as np

    from speech_b200.agents.transport import WebsocketAudioTransport, float_to_pcm16, pcm16_to_float
    from speech_b200.agents.voice_agent import build_voice_agent

    x = np.linspace(-1, 1, 9, dtype=np.float32)
    assert np.abs(pcm16_to_float(float_to_pcm16(x)) - x).max() < 1e-4

    class FakeWS:
        def __init__(self, incoming):
            self.incoming, self.sent_text, self.sent_bytes = list(incoming), [], []
        async def receive(self):
            return self.incoming.pop(0) if self.incoming else {"type": "websocket.disconnect"}
        async def send_text(self, t): self.sent_text.append(json.loads(t))
        async def send_bytes(self, b): self.sent_bytes.append(b)

    sr = 16000
    rng = np.random.default_rng(0)
    speech = (0.2 * rng.standard_normal(int(0.8 * sr))).astype(np.float32)
    silence = np.zeros(int(1.0 * sr), np.float32)
    audio = np.concatenate([speech, silence])
    msgs = [{"type": "message", "text": json.dumps({"type": "config", "sample_rate": sr})}]
    for i in range(0, len(audio), 1000):                       # odd chunking on purpose: the transport re-frames to 80 ms
        msgs.append({"type": "message", "bytes": float_to_pcm16(audio[i:i + 1000])})
    msgs.append({"type": "message", "text": "not json"})
    msgs.append({"type": "message", "text": json.dumps({"type": "end"})})
    seen = []
    def stt(chunk):
        seen.append(len(chunk))
        return ("hello there" if float(np.sqrt((chunk ** 2).mean())) > 0.01 else None), False
    agent = build_voice_agent(stt, lambda hist: "hi " + hist[-1]["content"], lambda text: (np.full(4410, 0.1, np.float32), 22050),
                              speech_threshold=0.01, max_silence=0.4)
    ws = FakeWS(msgs)
    asyncio.run(WebsocketAudioTransport(agent, sr, frame_ms=80.0, tts_chunk_ms=50.0).serve(ws))
    assert set(seen) == {1280}                                    # every pipeline frame is 80 ms
    kinds = [e["type"] for e in ws.sent_text]
    assert "user_started" in kinds and "user_stopped" in kinds and "error" in kinds and kinds[-1] == "end"
    finals = [e for e in ws.sent_text if e["type"] == "transcript" and e["final"]]
    assert finals and finals[0]["text"] == "hello there"
    assert any(e["type"] == "bot_text" and e["text"] == "hi hello there" for e in ws.sent_text)
    assert {"type": "audio_format", "sample_rate": 22050} in ws.sent_text
    pcm = b"".join(ws.sent_bytes)
    assert len(pcm) == 4410 * 2 and len(ws.sent_bytes) == 5        # 200 ms of speech in packets of 1102 samples (50 ms)
    # the example server builds its FastAPI app with fallbacks for absent models
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "voice_agent", "server.py")
    spec = importlib.util.spec_from_file_location("va_server", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    from speech_b200.core.config import OmegaConf
    cfg = OmegaConf.create(mod.DEFAULTS)
    app = mod.build_app(cfg)
    assert any(getattr(r, "path", "") == "/ws" for r in app.routes) and any(getattr(r, "path", "") == "/health" for r in app.routes)
    step = mod.make_stt(cfg)
    assert step(speech[:1280]) == ("(speech)", False) and step(silence[:1280]) == (None, False)
    assert mod.make_llm(cfg)([{"role": "user", "content": "ping"}]) == "You said: ping"
    wav, rate = mod.make_tts(cfg)("two words")
    assert rate == 22050 and len(wav) == 2 * (int(0.12 * 22050) + int(0.05 * 22050))


def test_ctc_segmentation_finds_utterances_inside_a_long_recording(tmp_path):
    import json

    import numpy as np

    from speech_b200.data.audio_to_text import save_wav
    from speech_b200.decoding.ctc_segmentation import add_metrics, ctc_segment, cut_audio, filter_manifest, read_segments, split_text, write_segments

    orig, norm = split_text("Mr. Smith (laughs) paid 3 dollars.  Then he left!  A very long sentence that goes on, and on and on without end, yes.",
                            list("abcdefghijklmnopqrstuvwxyz' "), max_length=8, number_to_words=lambda d: {"3": "three"}[d])
    assert norm[0] == "mister smith paid three dollars" and norm[1] == "then he left" and len(norm) == 4 and orig[1] == "Then he left!"
    assert norm[2].endswith("goes on") and all(len(n.split()) <= 8 for n in norm)

    # synthetic posteriors: 40 frames of noise, utterance A, 30 frames of noise, utterance B (poorly matching), 25 frames of noise
    V, blank = 6, 5
    rng = np.random.default_rng(0)
    utt = [[0, 1, 2, 1], [3, 4, 3]]

    def render(tokens, conf):
        rows = []
        for t in tokens:
            for _ in range(3):
                r = np.full(V, (1 - conf) / (V - 1))
                r[t] = conf
                rows.append(r)
            r = np.full(V, 0.02)
            r[blank] = 0.9
            rows.append(r)
        return rows

    def noise(n):
        r = np.full((n, V), 0.02)
        r[:, blank] = 0.9
        return list(r)

    probs = np.array(noise(40) + render(utt[0], 0.9) + noise(30) + render(utt[1], 0.3) + noise(25))
    probs = probs / probs.sum(-1, keepdims=True)
    segs = ctc_segment(torch.tensor(np.log(probs)), utt, blank, frame_duration=0.04, score_window=6, texts=["a b c b", "d e d"])
    assert abs(segs[0].start - 40 * 0.04) <= 0.04 and abs(segs[0].end - 55 * 0.04) <= 0.08
    assert abs(segs[1].start - 86 * 0.04) <= 0.04 and segs[1].end <= (86 + 12) * 0.04 + 1e-6
    assert segs[0].score > -0.5 and segs[1].score < segs[0].score - 0.5          # the badly matching utterance scores low

    wav = tmp_path / "long.wav"
    save_wav(str(wav), (0.1 * rng.standard_normal(int(123 * 0.04 * 16000))).astype(np.float32), 16000)
    seg_file = tmp_path / "long_segments.txt"
    write_segments(str(seg_file), str(wav), segs, ["A b c b.", "D e d!"])
    path, back, orig2 = read_segments(str(seg_file))
    assert path == str(wav) and orig2 == ["A b c b.", "D e d!"] and back[0].text == "a b c b"
    manifests = cut_audio(str(seg_file), str(tmp_path / "out"), threshold=-0.8)
    rows = {k: [json.loads(l) for l in open(p)] for k, p in manifests.items()}
    assert len(rows["clips"]) == 1 and len(rows["low_score_clips"]) == 1 and len(rows["deleted_clips"]) == 3
    assert abs(rows["clips"][0]["duration"] - (segs[0].end - segs[0].start)) < 0.01 and os.path.exists(rows["clips"][0]["audio_filepath"])
    total = sum(r["duration"] for rs in rows.values() for r in rs)
    assert abs(total - 123 * 0.04) < 0.05                                          # nothing of the recording is lost
    m2, m3 = str(tmp_path / "m2.json"), str(tmp_path / "m3.json")
    both = tmp_path / "both.json"
    both.write_text(open(manifests["clips"]).read() + open(manifests["low_score_clips"]).read())
    got = add_metrics(str(both), m2, transcribe=lambda paths: ["a b c b", "x y z"])
    assert got[0]["WER"] == 0.0 and got[1]["WER"] == 100.0 and got[1]["start_CER"] > 0
    kept, dropped = filter_manifest(m2, m3, min_duration=0.1)
    assert kept > 0 and dropped > 0 and len(open(m3).read().splitlines()) == 1


def test_extra_data_tools(tmp_path):
    import json
    import tarfile

    import numpy as np

    from speech_b200.data import tools_extra as T
    from speech_b200.data.audio_to_text import load_audio, read_manifest, save_wav, write_manifest

    sr = 16000
    rng = np.random.default_rng(0)
    for spk in ("s1", "s2"):
        os.makedirs(tmp_path / "corpus" / spk / "wav", exist_ok=True)
    files = []
    for spk, n in (("s1", 4), ("s2", 2)):
        for k in range(n):
            p = tmp_path / "corpus" / spk / f"{spk}_{k}.wav"
            save_wav(str(p), (0.1 * rng.standard_normal(sr // 2 * (k + 1))).astype(np.float32), sr)
            files.append(str(p))
    # Kaldi directory with segments
    kd = tmp_path / "kaldi"
    os.makedirs(kd)
    (kd / "wav.scp").write_text(f"rec1 {files[3]}\nrec2 {files[5]}\n")
    (kd / "text").write_text("u1 hello world\nu2 good bye\nu3 again\n")
    (kd / "segments").write_text("u1 rec1 0.0 0.8\nu2 rec1 1.0 1.9\nu3 rec2 0.1 0.6\n")
    (kd / "utt2spk").write_text("u1 alice\nu2 alice\nu3 bob\n")
    assert T.kaldi2json(str(kd), str(tmp_path / "k.json")) == 3
    rows = read_manifest(str(tmp_path / "k.json"))
    assert rows[1]["offset"] == 1.0 and rows[1]["duration"] == 0.9 and rows[2]["speaker"] == "bob" and rows[0]["text"] == "hello world"
    (kd / "wav.scp").write_text("rec1 sox x.sph -t wav - |\n")
    with pytest.raises(ValueError):
        T.kaldi2json(str(kd), str(tmp_path / "k2.json"))
    # speaker manifests
    ntr, ndev = T.filelist_to_manifest(files, str(tmp_path / "spk.json"), id_index=-2, split_fraction=0.5)
    assert (ntr, ndev) == (3, 3) and {r["label"] for r in read_manifest(str(tmp_path / "spk_dev.json"))} == {"s1", "s2"}
    assert T.filelist_to_manifest(files, str(tmp_path / "spk3.json"), min_spkrs_count=3) == (4, 0)
    rttm = tmp_path / "s1_0.rttm"
    rttm.write_text("SPEAKER s1_0 1 0.0 0.2 <NA> <NA> A <NA> <NA>\nSPEAKER s1_0 1 0.2 0.2 <NA> <NA> B <NA> <NA>\n")
    assert T.pathfiles_to_diarize_manifest(files[:2], str(tmp_path / "diar.json"), rttm_paths=[str(rttm)], add_duration=True) == 2
    d = read_manifest(str(tmp_path / "diar.json"))
    assert d[0]["num_speakers"] == 2 and d[0]["rttm_filepath"] == str(rttm) and d[1]["rttm_filepath"] is None and d[0]["duration"] == 0.5
    # noise at a given SNR
    write_manifest(str(tmp_path / "clean.json"), [{"audio_filepath": files[1], "duration": 1.0, "text": "a"}])
    noise = tmp_path / "noise.wav"
    save_wav(str(noise), (0.05 * rng.standard_normal(3000)).astype(np.float32), sr)
    write_manifest(str(tmp_path / "noise.json"), [{"audio_filepath": str(noise), "duration": 3000 / sr}])
    outs = T.add_noise(str(tmp_path / "clean.json"), str(tmp_path / "noise.json"), str(tmp_path / "noisy"), snrs=[0, 20])
    x = load_audio(files[1])
    for mp, snr in zip(outs, (0, 20)):
        y = load_audio(read_manifest(mp)[0]["audio_filepath"])
        got = 10 * np.log10(np.mean(x ** 2) / np.mean((y - x) ** 2))
        assert abs(got - snr) < 0.7
    # code switching
    write_manifest(str(tmp_path / "en.json"), [{"audio_filepath": f, "duration": 0.5 * (k + 1), "text": f"en {k}"} for k, f in enumerate(files[:4])])
    write_manifest(str(tmp_path / "es.json"), [{"audio_filepath": f, "duration": 0.5 * (k + 1), "text": f"es {k}"} for k, f in enumerate(files[4:])])
    n = T.code_switching_manifest(str(tmp_path / "en.json"), str(tmp_path / "es.json"), str(tmp_path / "cs.json"), "en", "es", max_sample_duration=4.0,
                                  min_sample_duration=2.0, dataset_size_hours=20 / 3600)
    cs = [json.loads(l) for l in open(tmp_path / "cs.json")]
    assert n == len(cs) >= 5 and all(2.0 <= c["duration"] <= 4.0 for c in cs) and {l for c in cs for l in c["lang_ids"]} == {"en", "es"}
    m = T.code_switching_audio(str(tmp_path / "cs.json"), str(tmp_path / "cs_audio"), str(tmp_path / "cs_out.json"))
    r0 = read_manifest(str(tmp_path / "cs_out.json"))[0]
    assert m == n and r0["duration"] > cs[0]["duration"] and len(r0["word_lang_ids"]) == len(r0["text"].split())
    # end of utterance labels, keyword scores, confidence metrics
    write_manifest(str(tmp_path / "eou.json"), [{"audio_filepath": files[0], "duration": 1, "text": "Uh-huh"}, {"audio_filepath": files[0], "duration": 1, "text": "I'll go now!"},
                                                {"audio_filepath": files[0], "duration": 1, "text": "??"}])
    assert T.clean_eou_manifest(str(tmp_path / "eou.json"), str(tmp_path / "eou_clean.json")) == 2
    assert T.add_eob_labels(str(tmp_path / "eou_clean.json"), str(tmp_path / "eou_lab.json")) == (1, 1)
    assert [r["eou_label"] for r in read_manifest(str(tmp_path / "eou_lab.json"))] == ["<EOB>", "<EOU>"]
    ks = T.keyword_fscore([{"text": "call nvidia and then call nvidia", "pred_text": "call in video and then call nvidia"},
                           {"text": "no key here", "pred_text": "nvidia here"}], ["nvidia", "call"])
    assert (ks["tp"], ks["fn"], ks["fp"]) == (3, 1, 1) and ks["precision"] == 0.75 and ks["recall"] == 0.75
    good = T.confidence_benchmark([0.9, 0.8, 0.95, 0.2, 0.1, 0.85], [True, True, True, False, False, True])
    bad = T.confidence_benchmark([0.5] * 6, [True, True, True, False, False, True])
    assert good["auc_roc"] == 1.0 and good["auc_nt"] == pytest.approx(1.0) and good["nce"] > 0.5 > bad["nce"] and good["ece"] < bad["ece"] + 0.2
    # token bins: equal token mass per bucket, 2-D sub-buckets
    counts = [10] * 90 + [100] * 9 + [1000]
    assert T.estimate_token_bins(counts, 3) == [100, 1000] and T.estimate_token_bins(counts, 2, max_tokens=100) == [10, 100]
    two = T.estimate_token_bins([10, 10, 10, 10, 20, 20], 2, num_subbuckets=2, second_dim=[1, 3, 5, 7, 9, 11])
    assert two == [(10, 3), (10, 7), (20, 9), (20, 11)]
    convs = [{"id": f"c{k}", "conversations": [{"from": "User", "type": "audio", "value": files[k], "duration": 0.5}, {"from": "Assistant", "type": "text", "value": "ok"}]}
             for k in range(3)]
    shards = T.export_conversations_to_tar(convs, str(tmp_path / "tars"), shard_size=2)
    assert len(shards) == 2
    with tarfile.open(shards[0]) as tf:
        names = tf.getnames()
        assert names == ["c0_0.wav", "c0.json", "c1_0.wav", "c1.json"]
        assert json.load(tf.extractfile("c0.json"))["conversations"][0]["value"] == "c0_0.wav"
    # pseudo-label merge
    write_manifest(str(tmp_path / "pred_rank0.json"), [{"audio_filepath": files[0], "pred_text": "new zero"}])
    write_manifest(str(tmp_path / "pred_rank1.json"), [{"audio_filepath": files[1], "pred_text": "new one"}])
    write_manifest(str(tmp_path / "src.json"), [{"audio_filepath": files[0], "duration": 1, "text": "old"}, {"audio_filepath": files[2], "duration": 1, "text": "untouched"}])
    out = T.write_transcribed_files(str(tmp_path / "pred_rank*.json"), [str(tmp_path / "src.json")])
    merged = read_manifest(out[0])
    assert len(merged) == 1 and merged[0]["text"] == "new zero" and merged[0]["orig_text"] == "old"


def test_asr_dataset_factories_tarred_noise_feature_and_record_datasets(tmp_path):
    """Tarred audio with scatter / replicate sharding and a shuffle buffer, bucket chains, config factories, audio+noise items,
    feature manifests gated by RTTM, record datasets and the prediction writer."""
    import json
    import tarfile

    import numpy as np
    import torch

    from speech_b200.data import asr_datasets_extra as X
    from speech_b200.data.audio_to_text import save_wav

    labels = list(" abcdefghijklmnopqrstuvwxyz'")
    rng = np.random.RandomState(0)
    entries, tars = [], []
    for s in range(2):
        tar = tmp_path / f"audio_{s}.tar"
        with tarfile.open(tar, "w") as tf:
            for k in range(3):
                name = f"utt{s}{k}.wav"
                p = tmp_path / name
                save_wav(str(p), (rng.randn(1600 * (k + 2)) * 0.1).astype(np.float32))
                tf.add(p, arcname=name)
                entries.append({"audio_filepath": name, "duration": 0.1 * (k + 2), "text": "ab" * (k + 1), "label": "x" if k else "y"})
        tars.append(str(tar))
    man = tmp_path / "tarred.json"
    man.write_text("".join(json.dumps(e) + "\n" for e in entries))
    brace = str(tmp_path / "audio__OP_0..1_CL_.tar")

    ds = X.TarredAudioToCharDataset(brace, str(man), labels=labels, return_sample_id=True)
    got = list(ds)
    assert len(got) == 6 and [g[3] for g in got] == [2, 4, 6, 2, 4, 6] and got[1][0].shape[0] == 4800
    r0 = list(X.TarredAudioToCharDataset(brace, str(man), labels=labels, world_size=2, global_rank=0, return_sample_id=True))
    r1 = list(X.TarredAudioToCharDataset(brace, str(man), labels=labels, world_size=2, global_rank=1, return_sample_id=True))
    assert sorted(g[4] for g in r0) == [0, 1, 2] and sorted(g[4] for g in r1) == [3, 4, 5]
    rep = X.TarredAudioToCharDataset(brace, str(man), labels=labels, world_size=2, global_rank=1, shard_strategy="replicate")
    assert len(list(rep)) == 6 and len(rep) == 6
    sh = X.TarredAudioToCharDataset(brace, str(man), labels=labels, shuffle_n=4, return_sample_id=True)
    order = [g[4] for g in sh]
    assert sorted(order) == list(range(6)) and order != list(range(6))
    a, al, t, tl = ds.collate_fn([g[:4] for g in got[:3]])
    assert a.shape == (3, 6400) and t.shape == (3, 6)
    with pytest.raises(ValueError):
        X.shard_filepaths(tars, "scatter", world_size=3, global_rank=0)

    cl = X.TarredAudioToSpeechLabelDataset(brace, str(man), labels=["x", "y"], window_length_in_sec=0.1, shift_length_in_sec=0.1)
    xs, xl, ys, yl = cl.collate_fn(list(cl)[:2])
    assert xs.shape == (2 + 3, 1600) and ys.tolist() == [1, 1, 0, 0, 0]

    # buckets ---------------------------------------------------------------------------------------------------------
    assert X.convert_to_config_list("a,b") == [["a", "b"]] and X.convert_to_config_list([["a"], ["b"]]) == [["a"], ["b"]]
    with pytest.raises(ValueError):
        X.convert_to_config_list([])
    assert X.calc_bucketing_batch_sizes({"bucketing_batch_size": 2, "batch_size": 1}, 3) == [6, 4, 2]
    assert X.calc_bucketing_batch_sizes({"bucketing_batch_size": [8, 4], "batch_size": 1, "bucketing_weights": [2, 1]}, 3) == [8, 8, 4]
    with pytest.raises(ValueError):
        X.calc_bucketing_batch_sizes({"bucketing_batch_size": 2, "batch_size": 4}, 3)
    cfg = {"tarred_audio_filepaths": [[tars[0]], [tars[1]]], "manifest_filepath": [[str(man)], [str(man)]], "labels": labels, "batch_size": 1,
           "bucketing_batch_size": 1, "bucketing_strategy": "fixed_order", "is_tarred": True, "shuffle": False}
    chain = X.get_audio_to_text_char_dataset_from_config(cfg)
    groups = list(chain)
    assert [len(g) for g in groups] == [2, 1, 1, 1, 1]            # bucket 0 in pairs, bucket 1 one by one
    assert chain.datasets[0].collate_fn([groups[0]])[0].shape[0] == 2
    rnd = X.get_chain_dataset([ds, ds, ds], {"bucketing_strategy": "synced_randomized", "batch_size": 1})
    assert isinstance(rnd, X.RandomizedChainDataset) and len(list(rnd)) == 18
    with pytest.raises(ValueError):
        X.get_chain_dataset([ds, ds], {"bucketing_strategy": "nope", "batch_size": 1})

    # plain / concat factories -----------------------------------------------------------------------------------------
    plain = tmp_path / "plain.json"
    plain.write_text("".join(json.dumps({**e, "audio_filepath": str(tmp_path / e["audio_filepath"])}) + "\n" for e in entries))
    d = X.get_audio_to_text_char_dataset_from_config({"manifest_filepath": str(plain), "labels": labels, "return_sample_id": True})
    assert len(d) == 6 and d[2][3] == 6
    cc = X.get_audio_to_text_char_dataset_from_config({"manifest_filepath": [str(plain), str(plain)], "labels": labels, "is_concat": True,
                                                       "concat_sampling_technique": "round-robin"})
    assert len(list(cc)) == 12
    assert X.get_audio_to_text_char_dataset_from_config({"manifest_filepath": None, "labels": labels}) is None
    mc, dc = {"sample_rate": 8000, "labels": None}, {"sample_rate": 16000}
    X.inject_dataloader_value_from_model_config(mc, dc, "sample_rate")
    X.inject_dataloader_value_from_model_config(mc, dc, "labels")
    assert dc == {"sample_rate": 8000}

    # prediction writer -------------------------------------------------------------------------------------------------
    w = X.ASRPredictionWriter(d, str(tmp_path / "pred.json"))
    w.write_on_batch_end(prediction=[(0, "hello"), (2, type("H", (), {"text": "world", "timestamp": None, "token_confidence": None})())])
    assert w.close_output_file() == 2
    lines = [json.loads(l) for l in open(tmp_path / "pred.json")]
    assert lines[0]["pred_text"] == "hello" and lines[1]["pred_text"] == "world" and lines[1]["text"] == "ababab"

    # audio + noise ------------------------------------------------------------------------------------------------------
    nz = X.AudioNoiseDataset(manifest_filepath=str(plain), noise_manifest=str(plain), min_audio_len_secs=0.3)
    item = nz[0]
    assert len(item.audio) == 4800 and torch.equal(item.audio[3200:], item.audio[:1600])
    assert torch.allclose(item.noisy_audio, item.audio + item.noise) and float(item.noise.abs().sum()) > 0
    batch = nz.collate_fn([nz[0], nz[2]])
    assert batch.audio.shape == (2, 6400) and batch.noisy_audio_len.tolist() == [4800, 6400]
    silent = X.AudioNoiseDataset(manifest_filepath=str(plain))[1]
    assert float(silent.noise.abs().sum()) == 0.0
    x = torch.arange(3.0)
    assert X.pad_audio(x, 7, "repeat").tolist() == [0, 1, 2, 0, 1, 2, 0] and X.pad_audio(x, 5, "zero").tolist() == [0, 1, 2, 0, 0]
    wn, wl = X.load_noise_audio({"audio_filepath": str(tmp_path / "missing.wav"), "duration": 1.0}, 16000, 800)
    assert wn.shape == (800,) and 0 < float(wn.abs().max()) < 0.05
    tn = list(X.get_audio_noise_dataset_from_config({"manifest_filepath": str(man), "tarred_audio_filepaths": brace, "is_tarred": True,
                                                     "noise_manifest": str(plain), "batch_size": 1}))
    assert len(tn) == 6 and isinstance(tn[0], X.AudioNoiseItem)

    # feature manifests with RTTM gating -----------------------------------------------------------------------------------
    feat = torch.arange(80.0).reshape(1, 80).repeat(4, 1)
    np.save(tmp_path / "f.npy", feat.numpy())
    (tmp_path / "f.rttm").write_text("SPEAKER f 1 0.10 0.20 <NA> <NA> s <NA> <NA>\nSPEAKER f 1 0.50 0.10 <NA> <NA> s <NA> <NA>\n")
    fm = tmp_path / "feat.json"
    fm.write_text(json.dumps({"feature_file": str(tmp_path / "f.npy"), "rttm_filepath": str(tmp_path / "f.rttm"), "duration": 0.8, "text": "abc"}) + "\n")
    fd = X.get_feature_char_dataset({"manifest_filepath": str(fm), "labels": labels, "use_rttm": True, "rttm_mode": "drop"})
    f, fl, y, yl = fd[0]
    assert fl == 30 and f[0, :20].tolist() == list(range(10, 30)) and f[0, 20:].tolist() == list(range(50, 60)) and y.tolist() == [1, 2, 3]
    fmask = X.FeatureToCharDataset(str(fm), labels=labels, use_rttm=True, rttm_mode="mask")[0][0]
    assert fmask.shape == (4, 80) and float(fmask[0, 0]) == pytest.approx(-16.635) and float(fmask[0, 15]) == 15.0
    F, FL, Y, YL = fd.collate_fn([fd[0], fd[0]])
    assert F.shape == (2, 4, 30) and Y.shape == (2, 3)

    # record datasets ---------------------------------------------------------------------------------------------------------
    recs = [{"audio": {"array": rng.randn(8000).astype(np.float32), "sampling_rate": 8000}, "text": "Ab, c!", "id": f"r{k}"} for k in range(5)]
    hd = X.get_hf_audio_to_text_char_dataset({"labels": labels, "normalize_text": True, "return_sample_id": True, "id_key": "id"}, records=recs)
    a0 = hd[1]
    assert a0[0].shape[0] == 16000 and a0[2].tolist() == [1, 2, 0, 3] and a0[4] == "r1"
    assert X.get_nested_dict_value(recs[0], "audio.sampling_rate") == 8000
    it0 = list(X.get_hf_audio_to_text_char_dataset({"labels": labels, "streaming": True, "return_sample_id": True}, world_size=2, global_rank=0, records=recs))
    it1 = list(X.get_hf_audio_to_text_char_dataset({"labels": labels, "streaming": True, "return_sample_id": True}, world_size=2, global_rank=1, records=recs))
    assert [s[4] for s in it0] == [0, 2, 4] and [s[4] for s in it1] == [1, 3]

    class Tok:
        bos_id, eos_id = 1, 2

        def text_to_ids(self, t):
            return [10 + len(w) for w in t.split()]

    hb = X.get_hf_audio_to_text_bpe_dataset({"use_start_end_token": True}, Tok(), records=recs)
    assert hb[0][2].tolist() == [1, 13, 12, 2]


def test_manifest_collections_parse_filter_and_index(tmp_path):
    import json

    from speech_b200.data import collections as C

    (tmp_path / "a.wav").write_bytes(b"")
    (tmp_path / "t.txt").write_text("from file\n")
    (tmp_path / "s.rttm").write_text("SPEAKER s 1 0.0 1.0 <NA> <NA> bob <NA> <NA>\nSPEAKER s 1 1.0 1.0 <NA> <NA> amy <NA> <NA>\nSPEAKER s 1 2.0 1.0 <NA> <NA> bob <NA> <NA>\n")
    man = tmp_path / "m.json"
    rows = [{"audio_filepath": "a.wav", "duration": 3.0, "text": "hello", "lang": "en", "offset": 1.0},
            {"audio_filename": "/abs/b.wav", "duration": 0.2, "text": "short"},
            {"audio_filepath": "c.wav", "duration": 2.0, "text_filepath": "t.txt", "speaker": 7},
            {"audio_filepath": "d.wav", "duration": 1.0, "normalized_text": "norm", "token_labels": [4, 5]}]
    man.write_text("".join(json.dumps(r) + "\n" for r in rows))
    parser = lambda t: [ord(c) - 96 for c in t if c.isalpha()]  # noqa: E731
    col = C.ASRAudioText(str(man), parser=parser, min_duration=0.5, do_sort_by_duration=True)
    assert [e.duration for e in col] == [1.0, 2.0, 3.0]
    assert col[2].audio_file == str(tmp_path / "a.wav") and col[2].text_tokens == [8, 5, 12, 12, 15] and col[2].lang == "en" and col[2].offset == 1.0
    assert col[1].text_raw == "from file" and col[1].speaker == 7 and col[0].text_tokens == [4, 5] and col[0].text_raw == "norm"
    idx = C.ASRAudioText(str(man), parser=parser, index_by_file_id=True, max_number=3)
    assert len(idx) == 3 and idx.mapping["c"] == [2]
    with pytest.raises(ValueError):
        C.parse_item(json.dumps({"text": "x", "duration": 1.0}), str(man))
    assert C.get_full_path("a.wav", str(man)) == str(tmp_path / "a.wav") and C.get_full_path("zz.wav", str(man)) == "zz.wav"
    assert [e.tokens for e in C.FromFileText(str(tmp_path / "t.txt"), parser)] == [[6, 18, 15, 13, 6, 9, 12, 5]]

    lm = tmp_path / "l.json"
    lm.write_text("".join(json.dumps(r) + "\n" for r in [{"audio_filepath": "a.wav", "duration": 1.0, "label": "yes"}, {"audio_filepath": "b.wav", "duration": 2.0, "command": "no"},
                                                       {"audio_filepath": "c.wav", "duration": 9.0, "target": "yes"}]))
    sl = C.ASRSpeechLabel(str(lm), max_duration=5.0, cal_labels_occurrence=True)
    assert [e.label for e in sl] == ["yes", "no"] and sl.uniq_labels == ["no", "yes"] and sl.labels_occurrence == {"yes": 2, "no": 1}
    reg = tmp_path / "r.json"
    reg.write_text(json.dumps({"audio_filepath": "a.wav", "duration": 1.0, "label": "0.5"}) + "\n")
    assert C.ASRSpeechLabel(str(reg), is_regression_task=True)[0].label == 0.5

    assert C.FeatureSequenceLabel.relative_speaker_parser("c a c b") == [0, 1, 0, 2]
    fm = tmp_path / "f.json"
    fm.write_text(json.dumps({"feature_filepath": "x.npy", "seq_label": "s2 s1 s2", "label": "0 1 1", "duration": 0.3, "text": "ab", "rttm_filepath": "s.rttm"}) + "\n")
    assert C.ASRFeatureSequenceLabel(str(fm))[0].seq_label == [0, 1, 0]
    fl = C.ASRFeatureLabel(str(fm), cal_labels_occurrence=True, delimiter=" ")
    assert fl[0].label == "0 1 1" and fl.labels_occurrence == {"0": 1, "1": 2}
    ft = C.ASRFeatureText(str(fm), parser=parser)
    assert ft[0].feature_file == "x.npy" and ft[0].rttm_file == str(tmp_path / "s.rttm") and ft[0].text_tokens == [1, 2]

    dm = tmp_path / "d.json"
    dm.write_text(json.dumps({"audio_filepath": "/x/s.wav", "duration": 3.0, "rttm_filepath": str(tmp_path / "s.rttm"), "offset": 1.5}) + "\n")
    tr = C.DiarizationSpeechLabel(str(dm))
    assert len(tr) == 1 and tr[0].target_spks == (0, 1) and tr[0].sess_spk_dict == {0: "bob", 1: "amy"} and tr[0].rttm_spk_digits == [0, 1]
    inf = C.DiarizationSpeechLabel(str(dm), clus_label_dict={"s": ["0 1 speaker_0", "1 2 speaker_1", "2 3 speaker_2"]}, pairwise_infer=True)
    assert [e.target_spks for e in inf] == [(0, 1), (0, 2), (1, 2)] and inf[0].clus_spk_digits == [0, 1, 2]
    e2e = C.EndtoEndDiarizationSpeechLabel(str(dm))
    assert e2e[0].uniq_id == "s_1500_3000" and e2e[0].rttm_file == str(tmp_path / "s.rttm")

    am = tmp_path / "au.json"
    am.write_text(json.dumps({"noisy": "n.wav", "clean": ["c1.wav", "c2.wav"], "extra": "e.wav", "duration": 2.0}) + "\n")
    ac = C.AudioCollection(str(am), {"input_signal": "noisy", "target_signal": "clean,extra"})
    assert ac[0].audio_files == {"input_signal": "n.wav", "target_signal": ["c1.wav", "c2.wav", "e.wav"]} and ac[0].offset == 0.0
    with pytest.raises(KeyError):
        C.AudioCollection(str(am), {"input_signal": "nope"})

    qm = tmp_path / "q.json"
    qm.write_text("".join(json.dumps(r) + "\n" for r in [{"audio_filepath": "a.wav", "duration": 1.0, "context": "transcribe", "answer": "hi"},
                                                       {"audio_filepath": "b.wav", "duration": 2.0, "text": "yo"},
                                                       {"context": "text only", "context_duration": 0.5, "answer": "ok"}]))
    q = C.SpeechLLMAudioTextCollection(str(qm))
    assert [(e.context, e.answer) for e in q] == [("transcribe", "hi"), ("what does this audio mean", "yo"), ("text only", "ok")] and q[2].audio_file is None
    (tmp_path / "ctx.txt").write_text("describe it\n")
    assert C.SpeechLLMAudioTextCollection(str(qm), context_file=str(tmp_path / "ctx.txt"), max_num_samples=2)[0].context == "describe it"


def test_text_adapters_typed_examples_prompt_formats_and_tar_writer(tmp_path):
    import json

    import numpy as np
    import torch

    from speech_b200.data import text_adapters as T
    from speech_b200.data.audio_to_text import save_wav
    from speech_b200.data.cuts import Cut
    from speech_b200.prompts import PromptFormatter

    class Tok:
        bos_id, eos_id, pad_id = 1, 2, 0

        def text_to_ids(self, t):
            return [3 + (ord(c) % 50) for c in t]

        def token_to_id(self, t):
            return 60

    prompt = PromptFormatter.resolve("plain")(Tok())
    (tmp_path / "a.txt").write_text("hello\nworld\n")
    (tmp_path / "b.txt").write_text("hallo\nwelt\n")
    (tmp_path / "q.txt").write_text("translate:\n")
    ex = list(T.LhotseTextAdapter(str(tmp_path / "a.txt"), language="en"))
    assert [e.text for e in ex] == ["hello", "world"] and ex[0].tokenize(Tok()).num_tokens == 5
    ex[0].apply_prompt_format(prompt)
    assert ex[0].input_length == 0 and ex[0].output_length == ex[0].total_length == 6 and bool(ex[0].mask.all())
    (tmp_path / "j.jsonl").write_text(json.dumps({"content": "abc", "k": 1}) + "\n")
    je = list(T.LhotseTextJsonlAdapter(str(tmp_path / "j.jsonl"), text_field="content"))
    assert je[0].text == "abc" and je[0].custom["k"] == 1

    pairs = list(T.LhotseTextPairAdapter(str(tmp_path / "a.txt"), str(tmp_path / "b.txt"), "en", "de", questions_path=str(tmp_path / "q.txt")))
    assert pairs[1].source.text == "world" and pairs[1].target.text == "welt" and pairs[1].question.text == "translate:" and pairs[1].target.language == "de"
    pairs[0].apply_prompt_format(prompt)
    assert pairs[0].output_length >= 5 and pairs[0].input_length >= len("translate: hello") and pairs[0].total_length == pairs[0].input_length + pairs[0].output_length
    with pytest.raises(ValueError):
        T.LhotseTextPairAdapter([str(tmp_path / "a.txt"), str(tmp_path / "b.txt")], str(tmp_path / "b.txt"))

    (tmp_path / "sft.jsonl").write_text(json.dumps({"system": "", "mask": "User", "conversations": [{"from": "User", "value": "hi"}, {"from": "Assistant", "value": "yo"}]}) + "\n")
    sft = list(T.NeMoSFTJsonlAdapter(str(tmp_path / "sft.jsonl")))[0]
    sft.apply_prompt_format(prompt)
    assert sft.data["conversations"][1]["value"] == "yo" and int(sft.mask.sum()) == sft.output_length and sft.input_length > 0

    # conversations: write tar shards, read them back ---------------------------------------------------------------
    rng = np.random.RandomState(0)
    for n in ("u1", "u2", "u3"):
        save_wav(str(tmp_path / f"{n}.wav"), (rng.randn(8000) * 0.1).astype(np.float32))
    convs = [T.NeMoMultimodalConversation(f"c{k}", [T.TextTurn("transcribe", "user"), T.AudioTurn(Cut(n, str(tmp_path / f"{n}.wav"), 0.25, offset=0.1), "user"),
                                                   T.TextTurn(f"answer {k}", "assistant")], token_equivalent_duration=0.08) for k, n in enumerate(("u1", "u2", "u3"))]
    assert convs[0].has_audio_turns and convs[0].has_text_turns and not convs[0].is_text_only and len(convs[0].list_cuts()) == 1
    assert convs[0].to_dict()["conversations"][1] == {"type": "audio", "from": "User", "duration": 0.25, "value": str(tmp_path / "u1.wav"), "offset": 0.1}
    convs[0].apply_prompt_format(prompt)
    n_audio = int(np.ceil(0.25 / 0.08)) - 1
    assert convs[0].total_length == len(convs[0].input_ids) + n_audio and convs[0].input_length == len(convs[0].context_ids) + n_audio
    assert convs[0].output_length == len(convs[0].answer_ids)
    out = tmp_path / "shards"
    with T.NeMoMultimodalConversationTarWriter(str(out), shard_size=2) as w:
        for c in convs:
            w.write(c)
    assert sorted(p.name for p in out.iterdir()) == ["audio_0.tar", "audio_1.tar", "manifest_0.jsonl", "manifest_1.jsonl"] and w.total == 3
    assert [n for n, _ in T.TarIterator(str(out / "audio_0.tar"))] == ["u1.wav", "u2.wav"]
    back = list(T.NeMoMultimodalConversationJsonlAdapter(str(out / "manifest__OP_0..1_CL_.jsonl"), tarred_audio_filepaths=str(out / "audio__OP_0..1_CL_.tar"),
                                                         token_equivalent_duration=0.08))
    assert [b.id for b in back] == ["c0", "c1", "c2"] and back[2].turns[2].value == "answer 2"
    a = back[1].turns[1]
    assert isinstance(a, T.AudioTurn) and a.cut.duration == pytest.approx(0.25) and len(a.cut.load_audio()) == 4000
    audio, lens, kept = T.collate_conversation_audio_fault_tolerant(back)
    assert audio.shape == (3, 4000) and len(kept) == 3
    bad = T.NeMoMultimodalConversation("bad", [T.AudioTurn(Cut("x", str(tmp_path / "missing.wav"), 1.0), "user")])
    audio, lens, kept = T.collate_conversation_audio_fault_tolerant([bad, back[0]])
    assert audio.shape == (1, 4000) and [k.id for k in kept] == ["c0"]

    (tmp_path / "sg.jsonl").write_text(json.dumps({"id": "s0", "sound": str(tmp_path / "u1.wav"), "duration": 0.5,
                                                    "conversations": [{"from": "human", "value": "what is said <sound> here"}, {"from": "gpt", "value": "words"}]}) + "\n")
    sg = list(T.NeMoMultimodalConversationShareGPTJsonlAdapter(str(tmp_path / "sg.jsonl")))[0]
    assert [type(t).__name__ for t in sg.turns] == ["TextTurn", "AudioTurn", "TextTurn", "TextTurn"] and sg.turns[3].role == "assistant"
    ids = T.default_multimodal_conversation_prompt_format_fn(sg, prompt)
    assert int(ids["mask"].sum()) == len(ids["answer_ids"])
