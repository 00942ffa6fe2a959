"""Input-source readers, sampling constraints and filters of the cut pipeline (CPU)."""
import gzip
import io
import json
import os
import tarfile

import numpy as np
import pytest
import torch

from speech_b200.data.audio_to_text import save_wav
from speech_b200.data.cuts import get_dataloader_from_cuts_config, parse_input_cfg
from speech_b200.data.sampling import (BucketingFilter, CERFilter, DurationFilter, FixedBucketBatchSizeConstraint2D,
                                       MultimodalFixedBucketBatchSizeConstraint2D, MultimodalSamplingConstraint, TokenCountFilter,
                                       TokenPerSecondFilter, TokenPerTokenFilter, ValidationStatusFilter, batches_from_constraint,
                                       find_smallest_bucket)
from speech_b200.data.sources import data_type_parser, known_data_types, measure_tokens, sharegpt_turns


def _wav(path, seconds, seed=0):
    x = (0.1 * np.random.default_rng(seed).standard_normal(int(16000 * seconds))).astype(np.float32)
    save_wav(str(path), x)
    return x


def _write_shar(d, n_shards=2, per_shard=3):
    """A Shar directory as Lhotse writes it: cuts.k.jsonl.gz + recording.k.tar with <id>.wav / <id>.json members."""
    os.makedirs(d, exist_ok=True)
    ids = []
    for k in range(n_shards):
        with gzip.open(os.path.join(d, f"cuts.{k:06d}.jsonl.gz"), "wt") as f, tarfile.open(os.path.join(d, f"recording.{k:06d}.tar"), "w") as tf:
            for j in range(per_shard):
                cid = f"utt-{k}-{j}"
                dur = 0.2 + 0.1 * j
                tmp = os.path.join(d, "tmp.wav")
                _wav(tmp, dur, seed=10 * k + j)
                data = open(tmp, "rb").read()
                os.remove(tmp)
                cut = {"id": cid, "start": 1.5, "duration": dur, "channel": 0, "type": "MonoCut",
                       "supervisions": [{"id": cid, "recording_id": cid, "start": 0.0, "duration": dur, "text": f"hello {k} {j}", "language": "en", "speaker": "s1"}],
                       "recording": {"id": cid, "sources": [{"type": "shar", "channels": [0], "source": ""}], "sampling_rate": 16000,
                                     "num_samples": int(dur * 16000), "duration": dur}}
                f.write(json.dumps(cut) + "\n")
                for name, payload in ((f"{cid}.wav", data), (f"{cid}.json", json.dumps(cut["recording"]).encode())):
                    ti = tarfile.TarInfo(name)
                    ti.size = len(payload)
                    tf.addfile(ti, io.BytesIO(payload))
                ids.append(cid)
    return ids


def test_lhotse_shar_and_lhotse_manifest(tmp_path):
    ids = _write_shar(str(tmp_path / "shar"))
    cuts = list(parse_input_cfg([{"type": "lhotse_shar", "shar_path": str(tmp_path / "shar"), "tags": {"corpus": "x"}}]))
    assert [c.id for c in cuts] == ids
    assert cuts[1].text == "hello 0 1" and cuts[1].lang == "en" and cuts[1].custom["corpus"] == "x"
    x = cuts[2].load_audio()
    assert abs(len(x) - int(0.4 * 16000)) <= 1 and cuts[2].offset == 0.0
    # shards are split over ranks
    r0 = [c.id for c in parse_input_cfg([{"type": "lhotse_shar", "shar_path": str(tmp_path / "shar")}], rank=0, world=2)]
    r1 = [c.id for c in parse_input_cfg([{"type": "lhotse_shar", "shar_path": str(tmp_path / "shar")}], rank=1, world=2)]
    assert r0 == ids[:3] and r1 == ids[3:]
    # through the loader config
    dl = get_dataloader_from_cuts_config({"shar_path": str(tmp_path / "shar"), "batch_size": 2, "labels": None}, labels=list(" abcdefghijklmnopqrstuvwxyz0123456789"))
    b = next(iter(dl))
    assert b[0].shape[0] == 2
    # a plain cut manifest pointing at files
    _wav(tmp_path / "a.wav", 0.5)
    with open(tmp_path / "cuts.jsonl", "w") as f:
        f.write(json.dumps({"id": "a", "start": 0.1, "duration": 0.3, "supervisions": [{"text": "x y", "start": 0, "duration": 0.3}],
                            "recording": {"sources": [{"type": "file", "source": "a.wav"}], "sampling_rate": 16000}}) + "\n")
    (c,) = list(parse_input_cfg([{"type": "lhotse", "cuts_path": str(tmp_path / "cuts.jsonl")}]))
    assert c.text == "x y" and abs(len(c.load_audio()) - 4800) <= 1


def test_text_sources(tmp_path):
    (tmp_path / "src.txt").write_text("ein hund\nzwei katzen\n")
    (tmp_path / "tgt.txt").write_text("a dog\ntwo cats\n")
    (tmp_path / "q.txt").write_text("Translate:\nIn English:\n")
    pairs = list(parse_input_cfg([{"type": "txt_pair", "source_paths": str(tmp_path / "src.txt"), "target_paths": str(tmp_path / "tgt.txt"),
                                   "source_language": "de", "target_language": "en", "questions_path": str(tmp_path / "q.txt")}]))
    assert [p.custom["source"] for p in pairs] == ["ein hund", "zwei katzen"] and pairs[1].custom["target"] == "two cats"
    assert pairs[0].custom["question"] in ("Translate:", "In English:") and pairs[0].custom["kind"] == "text_pair"
    assert measure_tokens(pairs[1]) == (2 + len(pairs[1].custom["question"].split()), 2)
    with open(tmp_path / "t.jsonl", "w") as f:
        f.write(json.dumps({"content": "one two three", "src": "web"}) + "\n")
    (t,) = list(parse_input_cfg([{"type": "txt_jsonl", "paths": str(tmp_path / "t.jsonl"), "text_field": "content", "language": "en"}]))
    assert t.text == "one two three" and t.custom["src"] == "web" and measure_tokens(t) == (3, 0)
    with open(tmp_path / "sft.jsonl", "w") as f:
        f.write(json.dumps({"conversations": [{"from": "User", "value": "hi there"}, {"from": "Assistant", "value": "hello to you too"}],
                            "mask": "User", "system": "be kind"}) + "\n")
    (s,) = list(parse_input_cfg([{"type": "nemo_sft_jsonl", "paths": str(tmp_path / "sft.jsonl")}]))
    assert s.custom["kind"] == "sft" and measure_tokens(s) == (2, 4)
    # non-finite text sources repeat
    it = iter(parse_input_cfg([{"type": "txt", "paths": str(tmp_path / "src.txt"), "force_finite": False}]))
    assert [next(it).text for _ in range(5)] == ["ein hund", "zwei katzen", "ein hund", "zwei katzen", "ein hund"]
    assert {"share_gpt", "lhotse_shar", "multimodal_conversation", "parquet", "txt_pair"} <= set(known_data_types())


def test_conversation_sources(tmp_path):
    _wav(tmp_path / "q1.wav", 0.4)
    _wav(tmp_path / "q2.wav", 0.8)
    with open(tmp_path / "conv.jsonl", "w") as f:
        f.write(json.dumps({"id": "c1", "conversations": [
            {"from": "User", "type": "audio", "value": "q1.wav", "duration": 0.4},
            {"from": "Assistant", "type": "text", "value": "four words right here"}]}) + "\n")
    (c,) = list(parse_input_cfg([{"type": "multimodal_conversation", "manifest_filepath": str(tmp_path / "conv.jsonl"), "audio_locator_tag": "<a>",
                                  "token_equivalent_duration": 0.08, "tags": {"system_prompt": "sys", "context": "Transcribe this"}}]))
    t = c.custom["turns"]
    assert [x["role"] for x in t] == ["system", "user", "user", "assistant"] and t[1]["value"] == "Transcribe this"
    assert os.path.isabs(t[2]["value"]) and abs(c.duration - 0.4) < 1e-9
    assert measure_tokens(c) == (1 + 2 + 5, 4)
    # ShareGPT with a placeholder in the middle of a turn
    rec = {"id": "s1", "sound": "q2.wav", "duration": 0.8, "conversations": [{"from": "human", "value": "Listen: <sound> what is said?"},
                                                                             {"from": "gpt", "value": "nothing much"}]}
    turns = sharegpt_turns(rec)
    assert [(x["role"], x["type"]) for x in turns] == [("user", "text"), ("user", "audio"), ("user", "text"), ("assistant", "text")]
    with open(tmp_path / "sg.jsonl", "w") as f:
        f.write(json.dumps(rec) + "\n")
    (g,) = list(parse_input_cfg([{"type": "share_gpt", "manifest_filepath": str(tmp_path / "sg.jsonl"), "audio_locator_tag": "<a>", "slice_length": 0.5}]))
    a = [x for x in g.custom["turns"] if x["type"] == "audio"][0]
    assert a["duration"] == 0.5 and 0.0 <= a["offset"] <= 0.3 + 1e-9 and g.custom["conversation"]["conversations"][1]["type"] == "audio"
    # tarred conversations: the audio comes out of the tar in manifest order
    with tarfile.open(tmp_path / "audio_0.tar", "w") as tf:
        tf.add(str(tmp_path / "q1.wav"), arcname="q1.wav")
    (tc,) = list(parse_input_cfg([{"type": "multimodal_conversation", "manifest_filepath": str(tmp_path / "conv.jsonl"),
                                   "tarred_audio_filepaths": str(tmp_path / "audio_0.tar"), "audio_locator_tag": "<a>"}]))
    assert len(tc.custom["turns"][0]["audio"]) == 6400
    # plain audio manifest wrapped as a conversation
    with open(tmp_path / "m.json", "w") as f:
        f.write(json.dumps({"audio_filepath": str(tmp_path / "q1.wav"), "duration": 0.4, "text": "the answer"}) + "\n")
    (w,) = list(parse_input_cfg([{"type": "lhotse_as_conversation", "manifest_filepath": str(tmp_path / "m.json"), "tags": {"context": ["Transcribe"]}}]))
    assert [x["type"] for x in w.custom["turns"]] == ["text", "audio", "text"] and w.custom["turns"][-1]["value"] == "the answer"
    (d,) = list(parse_input_cfg([{"type": "nemo_tarred_to_duplex", "manifest_filepath": str(tmp_path / "m.json")}]))
    assert d.custom["duplex_turns"][1][0] == "agent" and d.duration > 0.4


def test_parquet_source_and_custom_parser(tmp_path):
    import pyarrow as pa
    import pyarrow.parquet as pq

    _wav(tmp_path / "a.wav", 0.25)
    data = open(tmp_path / "a.wav", "rb").read()
    pq.write_table(pa.table({"audio": [data, data], "text": ["one", "two"], "duration": [0.25, 0.25], "speaker": ["x", "y"]}), str(tmp_path / "d.parquet"))
    cuts = list(parse_input_cfg([{"type": "parquet", "manifest_filepath": str(tmp_path / "d.parquet")}]))
    assert [c.text for c in cuts] == ["one", "two"] and len(cuts[0].load_audio()) == 4000 and cuts[1].custom["speaker"] == "y"

    @data_type_parser("three_beeps")
    def _beeps(e, ctx):
        from speech_b200.data.cuts import Cut, CutSet
        return CutSet([Cut(f"b{i}", np.zeros(1600, np.float32), 0.1, text="beep") for i in range(3)])

    assert len(list(parse_input_cfg([{"type": "three_beeps"}]))) == 3
    with pytest.raises(ValueError, match="unsupported input_cfg type"):
        parse_input_cfg([{"type": "nope"}])


def test_constraints_and_filters():
    from speech_b200.data.cuts import Cut

    def audio(d, text=""):
        return Cut("a", None, d, text=text)

    def pair(ns, nt):
        return Cut("t", None, 0.0, text="", custom={"kind": "text_pair", "source": " ".join(["w"] * ns), "target": " ".join(["w"] * nt)})

    # 1-D and 2-D bucket search
    assert find_smallest_bucket([5.0, 10.0, 20.0], 7.0) == 1 and find_smallest_bucket([5.0, 10.0], 11.0) is None
    b2 = [(10, 5), (10, 10), (20, 12), (20, 18)]
    assert find_smallest_bucket(b2, (8, 4)) == 0 and find_smallest_bucket(b2, (8, 7)) == 1
    assert find_smallest_bucket(b2, (8, 11)) is None and find_smallest_bucket(b2, (8, 11), strict=False) == 2
    assert find_smallest_bucket(b2, (10, 10), max_ratio=[0.5] * 4) is None
    # token budget: audio of 0.8 s at 0.08 s/token is 10 tokens
    msc = MultimodalSamplingConstraint(token_equivalent_duration=0.08, batch_tokens=40)
    exs = [audio(0.8), audio(0.8), pair(10, 3), audio(0.8), audio(1.6), audio(1.6), pair(3, 1)]
    batches = batches_from_constraint(exs, msc)
    assert batches == [[0, 1, 2, 3], [4, 5], [6]]
    msc_total = MultimodalSamplingConstraint(token_equivalent_duration=0.08, measure_total_length=True)
    assert msc_total.measure_length(pair(10, 3)) == 13 and msc.measure_length(pair(10, 3)) == 10
    fb = FixedBucketBatchSizeConstraint2D([(1.0, 3), (1.0, 8), (2.0, 8)], [4, 2, 1])
    assert fb.select_bucket(audio(0.5, "a b c d")) == 1 and fb.select_bucket(audio(1.5, "a")) == 2 and fb.select_bucket(audio(3.0, "a")) is None
    assert batches_from_constraint([audio(0.5, "a b c d")] * 5, fb) == [[0, 1], [2, 3], [4]]
    assert BucketingFilter(fb)(audio(3.0, "a")) is False and BucketingFilter(fb)(audio(0.2, "a")) is True
    mfb = MultimodalFixedBucketBatchSizeConstraint2D([(10, 4), (10, 12), (30, 12)], [8, 4, 2], token_equivalent_duration=0.08)
    assert mfb.select_bucket(pair(9, 6)) == 1 and mfb.select_bucket(audio(1.6, "a b")) == 2
    # filters
    assert DurationFilter(0.5, 2.0)(audio(1.0)) and not DurationFilter(0.5, 2.0)(audio(2.5)) and DurationFilter(0.5, 2.0)(pair(1, 1))
    assert TokenCountFilter(2, 12, True)(pair(8, 3)) and not TokenCountFilter(2, 12, True)(pair(10, 3)) and TokenCountFilter(2, 12, False)(pair(10, 3))
    assert TokenPerSecondFilter(0.5, 4.0)(audio(1.0, "a b c")) and not TokenPerSecondFilter(0.5, 4.0)(audio(0.5, "a b c")) and TokenPerSecondFilter(0.5, 4.0)(pair(1, 9))
    assert TokenPerTokenFilter(0.5, 2.0)(pair(4, 4)) and not TokenPerTokenFilter(0.5, 2.0)(pair(2, 9)) and TokenPerTokenFilter(0.5, 2.0)(audio(1.0, "a"))
    c = audio(1.0); c.custom["validation_status"] = "fail"; c.custom["cer"] = 0.4
    assert not ValidationStatusFilter("pass")(c) and ValidationStatusFilter("pass")(audio(1.0))
    assert not CERFilter(0.2)(c) and CERFilter(0.5)(c) and CERFilter(None)(c)
    with pytest.raises(ValueError):
        TokenPerSecondFilter(5.0, 1.0)


def test_salm_loader_reads_a_mixture_of_sources(tmp_path):
    from speech_b200.speechlm.data import conversations_from_input_cfg

    _wav(tmp_path / "q1.wav", 0.4)
    with open(tmp_path / "m.json", "w") as f:
        f.write(json.dumps({"audio_filepath": str(tmp_path / "q1.wav"), "duration": 0.4, "text": "the answer"}) + "\n")
    (tmp_path / "s.txt").write_text("uno\n")
    (tmp_path / "t.txt").write_text("one\n")
    cfg = [{"type": "nemo", "manifest_filepath": str(tmp_path / "m.json"), "weight": 1.0},
           {"type": "txt_pair", "source_paths": str(tmp_path / "s.txt"), "target_paths": str(tmp_path / "t.txt"), "weight": 1.0}]
    convs = conversations_from_input_cfg(cfg, seed=1)
    kinds = sorted(tuple(t["type"] for t in c["conversations"]) for c in convs)
    assert kinds == [("audio", "text"), ("text", "text")]


def _canary_tokenizer():
    from speech_b200.tokenizers import CANARY_SPECIAL_TOKENIZER, CanaryTokenizer, CharTokenizer

    specials = ["<|nospeech|>", "<pad>", "<|endoftext|>", "<|startoftranscript|>", "<|pnc|>", "<|nopnc|>", "<|transcribe|>", "<|translate|>",
                "<|en|>", "<|de|>"]
    return CanaryTokenizer({CANARY_SPECIAL_TOKENIZER: CharTokenizer(specials), "en": CharTokenizer(list("abcdefghijklmnopqrstuvwxyz ")),
                            "de": CharTokenizer(list("abcdefghijklmnopqrstuvwxyzäöü "))})


def test_task_datasets_over_cuts_prompted_prompt_index_speaker_eou_diarization():
    from functools import partial

    from speech_b200.data.cuts import Cut
    from speech_b200.data.cuts_datasets import (DiarLabelCutsDataset, EOUCutsDataset, PromptedAudioToTextCutsDataset, PromptedAudioToTextMiniBatch,
                                                PromptIndexCutsDataset, SpeakerCutsDataset)
    from speech_b200.prompts import PromptFormatter

    tok = _canary_tokenizer()
    rng = np.random.default_rng(0)
    def wav(sec):
        return (0.1 * rng.standard_normal(int(16000 * sec))).astype(np.float32)
    cuts = [Cut("a", wav(0.5), 0.5, text="hallo welt", lang="de", custom={"source_lang": "en", "target_lang": "de", "pnc": "no"}),
            Cut("b", wav(0.8), 0.8, text="good day", lang="en", custom={"speaker": "s2"})]
    prompt = PromptFormatter.resolve("canary")(tokenizer=tok)
    ds = PromptedAudioToTextCutsDataset(cuts, tokenizer=tok, prompt=prompt, return_minibatch=True)
    mb = ds.collate_fn([ds[0], ds[1]])
    assert isinstance(mb, PromptedAudioToTextMiniBatch) and mb.audio.shape == (2, 12800) and mb.audio_lens.tolist() == [8000, 12800]
    sid = tok.spl_token_to_id
    assert mb.prompt[0, : mb.prompt_lens[0]].tolist() == [sid("startoftranscript"), sid("en"), sid("translate"), sid("de"), sid("nopnc")]
    assert mb.prompt[1, : mb.prompt_lens[1]].tolist() == [sid("startoftranscript"), sid("en"), sid("transcribe"), sid("en"), sid("pnc")]
    n0 = int(mb.prompted_transcript_lens[0])
    assert mb.prompted_transcript[0, n0 - 1] == sid("endoftext") and n0 == 5 + len("hallo welt") + 1
    assert torch.equal(mb.prompted_transcript[0, :5], mb.prompt[0, :5]) and mb.transcript_lens.tolist() == [len("hallo welt") + 1, len("good day") + 1]
    inp, out = mb.get_decoder_inputs_outputs()
    assert torch.equal(inp[:, 1:], out[:, :-1]) and ds.num_tokens(1) == 5 + len("good day") + 1
    tup = PromptedAudioToTextCutsDataset(cuts, tokenizer=tok, prompt=prompt).collate_fn([ds[0], ds[1]])
    assert len(tup) == 6 and torch.equal(tup[2], mb.prompted_transcript) and torch.equal(tup[5], mb.prompt_lens)
    # prompt index
    pi = PromptIndexCutsDataset(cuts, tokenizer=tok, prompt_dictionary={"en": 0, "de": 1, "fr": 2}, prompt_field="target_lang")
    b = pi.collate_fn([pi[0], pi[1]])
    assert b[4].tolist() == [[0.0, 1.0, 0.0], [1.0, 0.0, 0.0]]
    # speakers and activity
    multi = Cut("m", wav(1.0), 1.0, text="x", lang="en", custom={"speaker": "s1", "supervisions": [
        {"start": 0.0, "duration": 0.4, "speaker": "s1", "text": "x"}, {"start": 0.32, "duration": 0.4, "speaker": "s2", "text": "y"}]})
    sp = SpeakerCutsDataset([multi, cuts[1]], tokenizer=tok, frame_shift=0.08, max_speakers=3)
    b = sp.collate_fn([sp[0], sp[1]])
    assert b[4].tolist() == [0, 1] and b[5].shape == (2, 13, 3)
    assert b[5][0, :5, 0].tolist() == [1.0] * 5 and b[5][0, 4:9, 1].tolist() == [1.0] * 5 and float(b[5][0, :, 2].sum()) == 0.0
    dd = DiarLabelCutsDataset([multi], tokenizer=None, frame_shift=0.08, max_speakers=2)
    a, al, act, tl = dd.collate_fn([dd[0]])
    assert act.shape == (1, 13, 2) and tl.tolist() == [13] and float(act[0, 4, :].sum()) == 2.0        # overlap frame
    # end of utterance
    eo = EOUCutsDataset([Cut("e", wav(1.0), 1.0, text="ab", lang="en", custom={"sou_time": 0.16, "eou_time": 0.8}),
                         Cut("f", wav(1.0), 1.0, text="ab", lang="en", custom={"eou_time": 1.5, "is_backchannel": False})],
                        tokenizer=tok, eou_id=999, frame_shift=0.08)
    b = eo.collate_fn([eo[0], eo[1]])
    assert b[2][0, : b[3][0]].tolist()[-1] == 999 and 999 not in b[2][1].tolist()                      # the second utterance is cut short
    assert b[4][0].tolist() == [0, 0] + [1] * 8 + [2] * 3 and b[4][1].tolist() == [1] * 13
    padded = EOUCutsDataset([Cut("e", wav(1.0), 1.0, text="ab", lang="en")], tokenizer=tok, eou_id=999, pad_min=0.2, pad_max=0.4, seed=1)
    a, al, t, tl, lab = padded[0]
    assert int(al) > 16000 and lab[0] == 0 and lab[-1] == 2 and int((lab == 1).sum()) in (12, 13)
