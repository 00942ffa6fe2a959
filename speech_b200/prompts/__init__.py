"""Prompt formatters: turn-based templates with ``|slot|`` placeholders, encoded with a tokenizer.

``PromptFormatter.resolve(name)`` returns the class registered under ``NAME``; ``encode_dialog(turns)`` returns
``input_ids`` (full dialogue), ``context_ids`` (everything before the last assistant turn), ``answer_ids`` (the last
assistant turn) and ``mask`` (True on assistant tokens = loss positions), as in the reference
(``nemo/collections/common/prompts/formatter.py``).  Formats: ``canary`` (``prompts/canary.py:52,61``), ``canary2``
(``prompts/canary2.py:45-100``), ``qwen``, ``llama2``, ``llama3``, ``gemma``, ``mistral``, ``phi2``, ``nemotron_h``,
``nemotron_nano_v3``, ``t5nmt``, ``plain``.
"""
from __future__ import annotations

import re
from typing import Any, Dict, List, Optional, Type

import torch

BOS_SLOT = "|bos|"
EOS_SLOT = "|eos|"
CANARY_BOS = "<|startoftranscript|>"
CANARY_EOS = "<|endoftext|>"
CANARY2_BOCTX = "<|startofcontext|>"
CANARY_SPECIAL_TOKENIZER = "spl_tokens"

_REGISTRY: Dict[str, Type["PromptFormatter"]] = {}


class PromptFormatter:
    NAME: str = ""
    OUTPUT_ROLE: str = "assistant"
    INFERENCE_PREFIX: str = ""
    INSERT_BOS: bool = False
    INSERT_EOS: bool = False
    TEMPLATE: Dict[str, Dict[str, Any]] = {}

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        if cls.NAME:
            _REGISTRY[cls.NAME] = cls

    def __init__(self, tokenizer, defaults: Optional[List[dict]] = None):
        self.tokenizer = tokenizer
        self._defaults = defaults or []

    @classmethod
    def resolve(cls, name: str) -> Type["PromptFormatter"]:
        if name not in _REGISTRY:
            raise RuntimeError(f"Unknown prompt format: {name}. Available: {sorted(_REGISTRY)}")
        return _REGISTRY[name]

    @classmethod
    def get_roles(cls) -> List[str]:
        return list(cls.TEMPLATE.keys())

    @classmethod
    def get_slots(cls, role: str) -> Dict[str, Any]:
        return dict(cls.TEMPLATE[role].get("slots", {}))

    def get_default_dialog_slots(self) -> List[dict]:
        return [dict(t) for t in self._defaults]

    # ------------------------------------------------------------------ encoding
    def _tok(self, text: str, lang: Optional[str] = None) -> List[int]:
        tk = self.tokenizer
        if hasattr(tk, "langs"):
            return tk.text_to_ids(text, lang or tk.langs[0])
        return tk.text_to_ids(text)

    def _special(self, slot: str) -> List[int]:
        tk = self.tokenizer
        if slot == BOS_SLOT and getattr(tk, "bos_id", None) is not None and tk.bos_id >= 0:
            return [tk.bos_id]
        if slot == EOS_SLOT and getattr(tk, "eos_id", None) is not None and tk.eos_id >= 0:
            return [tk.eos_id]
        return []

    def fill(self, template: str, slots: Dict[str, Any]) -> str:
        def sub(m):
            key = m.group(1)
            if key not in slots:
                raise ValueError(f"Missing slot '{key}' for template '{template}' (got {list(slots)})")
            return str(slots[key])

        # slots look like |name|; special tokens such as <|im_start|> are left alone
        return re.sub(r"(?<!<)\|([A-Za-z_0-9]+)\|(?!>)", sub, template)

    def encode_turn(self, prompt_template: str, expected_slots: dict, slot_values: dict) -> List[int]:
        text = prompt_template.replace(BOS_SLOT, "").replace(EOS_SLOT, "")
        ids = self._special(BOS_SLOT) if prompt_template.startswith(BOS_SLOT) else []
        ids = ids + self._tok(self.fill(text, slot_values), slot_values.get("prompt_language"))
        if prompt_template.endswith(EOS_SLOT):
            ids = ids + self._special(EOS_SLOT)
        return ids

    def encode_dialog(self, turns: List[dict]) -> Dict[str, torch.Tensor]:
        if not turns:
            raise ValueError("Cannot encode an empty dialog")
        roles = self.get_roles()
        ids: List[int] = []
        mask: List[bool] = []
        turn_ids: List[List[int]] = []
        if self.INSERT_BOS:
            b = self._special(BOS_SLOT)
            ids += b
            mask += [False] * len(b)
        for turn in turns:
            role = turn["role"]
            if role not in roles:
                raise ValueError(f"Unknown role '{role}' for prompt format {self.NAME}; expected one of {roles}")
            tmpl = self.TEMPLATE[role]
            slots = dict(turn.get("slots", {}))
            missing = [s for s in tmpl.get("slots", {}) if s not in slots]
            if missing:
                raise ValueError(f"Turn with role '{role}' is missing slots {missing}")
            t_ids = self.encode_turn(tmpl["template"], tmpl.get("slots", {}), slots)
            turn_ids.append(t_ids)
            ids += t_ids
            mask += [role == self.OUTPUT_ROLE] * len(t_ids)
        out = {"input_ids": torch.tensor(ids, dtype=torch.long), "mask": torch.tensor(mask, dtype=torch.bool)}
        if turns[-1]["role"] == self.OUTPUT_ROLE:
            if self.INSERT_EOS:
                e = self._special(EOS_SLOT)
                ids += e
                mask += [True] * len(e)
                turn_ids[-1] = turn_ids[-1] + e
                out = {"input_ids": torch.tensor(ids, dtype=torch.long), "mask": torch.tensor(mask, dtype=torch.bool)}
            n_ans = len(turn_ids[-1])
            out["context_ids"] = out["input_ids"][: len(ids) - n_ans]
            out["answer_ids"] = out["input_ids"][len(ids) - n_ans:]
        else:
            if self.INFERENCE_PREFIX:
                pre = self._tok(self.INFERENCE_PREFIX)
                out["input_ids"] = torch.cat([out["input_ids"], torch.tensor(pre, dtype=torch.long)])
                out["mask"] = torch.cat([out["mask"], torch.zeros(len(pre), dtype=torch.bool)])
            out["context_ids"] = out["input_ids"]
        return out


class PlainPromptFormatter(PromptFormatter):
    NAME = "plain"
    INSERT_BOS, INSERT_EOS = True, True
    TEMPLATE = {"user": {"template": "|message|", "slots": {"message": str}},
                "assistant": {"template": "|message|", "slots": {"message": str}}}


class QwenPromptFormatter(PromptFormatter):
    NAME = "qwen"
    INFERENCE_PREFIX = "<|im_start|>assistant\n"
    TEMPLATE = {"system": {"template": "<|im_start|>system\n|message|<|im_end|>\n", "slots": {"message": str}},
                "user": {"template": "<|im_start|>user\n|message|<|im_end|>\n", "slots": {"message": str}},
                "assistant": {"template": "<|im_start|>assistant\n|message|<|im_end|>\n", "slots": {"message": str}}}


class Llama2PromptFormatter(PromptFormatter):
    NAME = "llama2"
    TEMPLATE = {"system_and_user": {"template": f"{BOS_SLOT}[INST] <<SYS>>\n|system|\n<</SYS>>\n\n|message| [/INST]",
                                    "slots": {"system": str, "message": str}},
                "user": {"template": f"{BOS_SLOT}[INST] |message| [/INST]", "slots": {"message": str}},
                "assistant": {"template": f"|message| {EOS_SLOT}", "slots": {"message": str}}}


class Llama3PromptFormatter(PromptFormatter):
    NAME = "llama3"
    INSERT_BOS = True
    INFERENCE_PREFIX = "<|start_header_id|>assistant<|end_header_id|>\n\n"
    TEMPLATE = {"system": {"template": "<|start_header_id|>system<|end_header_id|>\n\n|message|<|eot_id|>", "slots": {"message": str}},
                "user": {"template": "<|start_header_id|>user<|end_header_id|>\n\n|message|<|eot_id|>", "slots": {"message": str}},
                "assistant": {"template": "<|start_header_id|>assistant<|end_header_id|>\n\n|message|<|eot_id|>", "slots": {"message": str}}}


class GemmaPromptFormatter(PromptFormatter):
    NAME = "gemma"
    INSERT_BOS = True
    INFERENCE_PREFIX = "<start_of_turn>model\n"
    TEMPLATE = {"user": {"template": "<start_of_turn>user\n|message|<end_of_turn>\n", "slots": {"message": str}},
                "assistant": {"template": "<start_of_turn>model\n|message|<end_of_turn>\n", "slots": {"message": str}}}


class MistralPromptFormatter(PromptFormatter):
    NAME = "mistral"
    TEMPLATE = {"user": {"template": f"{BOS_SLOT}[INST] |message| [/INST]", "slots": {"message": str}},
                "assistant": {"template": f"|message|{EOS_SLOT}", "slots": {"message": str}}}


class Phi2PromptFormatter(PromptFormatter):
    NAME = "phi2"
    INFERENCE_PREFIX = "Output:"
    TEMPLATE = {"user": {"template": "Instruct: |message|\n", "slots": {"message": str}},
                "assistant": {"template": f"Output: |message|{EOS_SLOT}", "slots": {"message": str}}}


class NemotronHPromptFormatter(PromptFormatter):
    NAME = "nemotron_h"
    INFERENCE_PREFIX = "<SPECIAL_11>Assistant\n"
    TEMPLATE = {"system": {"template": "<SPECIAL_10>System\n|message|\n", "slots": {"message": str}},
                "user": {"template": "<SPECIAL_11>User\n|message|\n", "slots": {"message": str}},
                "assistant": {"template": "<SPECIAL_11>Assistant\n|message|\n<SPECIAL_12>\n", "slots": {"message": str}}}


class NemotronNanoV3PromptFormatter(QwenPromptFormatter):
    NAME = "nemotron_nano_v3"
    INFERENCE_PREFIX = "<|im_start|>assistant\n<think></think>"


class T5NMTPromptFormatter(PromptFormatter):
    NAME = "t5nmt"
    OUTPUT_ROLE = "assistant"
    TEMPLATE = {"user": {"template": "|target_lang| |message|", "slots": {"target_lang": str, "message": str}},
                "assistant": {"template": "|message|", "slots": {"message": str}}}

    def encode_turn(self, prompt_template, expected_slots, slot_values):
        sv = dict(slot_values)
        if "target_lang" in sv and not str(sv["target_lang"]).startswith("<"):
            sv["target_lang"] = f"<{sv['target_lang']}>"
        return super().encode_turn(prompt_template, expected_slots, sv)


# ---------------------------------------------------------------------------------------------------- Canary
PNC_TRUE = {"yes", "true", "True", "1", 1, True, "pnc", "<|pnc|>"}
TASK_TRANSLATE = {"ast", "translate", "<|translate|>", "s2t_translation"}


def _lang_token(v: str) -> str:
    return v if str(v).startswith("<|") else f"<|{v}|>"


class _CanaryBase(PromptFormatter):
    """Special tokens are encoded with the ``spl_tokens`` sub-tokenizer, free text with the language's tokenizer."""

    def _encode_mixed(self, text: str, lang: Optional[str]) -> List[int]:
        ids: List[int] = []
        for piece in re.split(r"(<\|[^|]*\|>)", text):
            if not piece:
                continue
            if piece.startswith("<|") and piece.endswith("|>"):
                ids += self.tokenizer.text_to_ids(piece, CANARY_SPECIAL_TOKENIZER)
            else:
                ids += self.tokenizer.text_to_ids(piece, lang)
        return ids


class CanaryPromptFormatter(_CanaryBase):
    NAME = "canary"
    TEMPLATE = {"user": {"template": f"{CANARY_BOS}|source_lang||task||target_lang||pnc|",
                         "slots": {"source_lang": str, "task": str, "target_lang": str, "pnc": str}},
                "assistant": {"template": f"|text|{CANARY_EOS}", "slots": {"text": str}}}

    def encode_turn(self, prompt_template, expected_slots, slot_values):
        sv = dict(slot_values)
        if "taskname" in sv and "task" not in sv:
            sv["task"] = sv.pop("taskname")
        lang = sv.get("prompt_language") or sv.get("target_lang") or sv.get("lang")
        if "source_lang" in sv:
            sv["source_lang"] = _lang_token(sv["source_lang"])
        if "target_lang" in sv:
            lang = str(sv["target_lang"]).strip("<|>")
            sv["target_lang"] = _lang_token(sv["target_lang"])
        if "task" in sv:
            sv["task"] = "<|translate|>" if sv["task"] in TASK_TRANSLATE else "<|transcribe|>"
        if "pnc" in sv:
            sv["pnc"] = "<|pnc|>" if sv["pnc"] in PNC_TRUE else "<|nopnc|>"
        return self._encode_mixed(self.fill(prompt_template, sv), lang)


class Canary2PromptFormatter(_CanaryBase):
    NAME = "canary2"
    TEMPLATE = {
        "user": {"template": f"{CANARY2_BOCTX}|decodercontext|{CANARY_BOS}|emotion||source_lang||target_lang||pnc||itn||timestamp||diarize|",
                 "slots": {"decodercontext": str, "emotion": str, "source_lang": str, "target_lang": str, "pnc": str, "itn": str,
                           "timestamp": str, "diarize": str}},
        "user_partial": {"template": f"{CANARY2_BOCTX}|decodercontext|{CANARY_BOS}", "slots": {"decodercontext": str}},
        "user_prefix": {"template": "|prefix|", "slots": {"prefix": str}},
        "assistant": {"template": f"|text|{CANARY_EOS}", "slots": {"text": str}},
    }
    _BOOL = {"pnc": ("<|pnc|>", "<|nopnc|>"), "itn": ("<|itn|>", "<|noitn|>"), "timestamp": ("<|timestamp|>", "<|notimestamp|>"),
             "diarize": ("<|diarize|>", "<|nodiarize|>")}

    def encode_turn(self, prompt_template, expected_slots, slot_values):
        sv = dict(slot_values)
        lang = sv.get("prompt_language") or (str(sv.get("target_lang", "")).strip("<|>") or None)
        for k in ("source_lang", "target_lang"):
            if k in sv:
                sv[k] = _lang_token(sv[k])
        for k, (yes, no) in self._BOOL.items():
            if k in sv and not str(sv[k]).startswith("<|"):
                sv[k] = yes if sv[k] in PNC_TRUE | {k} else no
        if "emotion" in sv and not str(sv["emotion"]).startswith("<|"):
            sv["emotion"] = f"<|emo:{sv['emotion']}|>"
        return self._encode_mixed(self.fill(prompt_template, sv), lang)


def get_prompt_format_fn(name: str):
    return PromptFormatter.resolve(name)
