"""Pick the best hyper-parameters of a sweep of domain-adaptation runs (adapters or fine-tuning) from a CSV of results.

Each row is one run: its hyper-parameters, the dataset group it adapted to, the WER on the new domain's test set and the WER on the original
domain's test set.  Two selections are reported per category (adapter position, or frozen module for fine-tuning):

* unconstrained — lowest mean WER on the new domain;
* constrained — highest mean ``Score = OriginalScale × AdaptWERR`` where ``AdaptWERR = max(baseline_new − WER_new, 0) / baseline_new`` is the relative
  gain on the new domain and ``OriginalScale = (D − min(D, |WER_orig − baseline_orig|)) / D`` scales it down linearly to zero as the original domain
  degrades by up to ``D`` (``--max_degradation``) absolute WER points.

Means are taken over the dataset groups for every hyper-parameter combination.  The scores are written back into the CSV.

python examples/asr/asr_adapters/scoring_and_analysis.py --csv results.csv --dataset_type_column Dataset --baselines baselines.json \
    [--finetuning] [--topk 3] [--show_analysis] [-cargs 'Adapter Dropout' 0.5] [-uargs 'Train Steps' 5000]
``baselines.json``: ``{"original": 5.1, "adapted": {"<dataset group>": 20.7, ...}}``.
(reference script: ``examples/asr/asr_adapters/scoring_and_analysis.py``)."""
import argparse
import json
from typing import Dict, List, Sequence, Tuple

import pandas as pd

TEST_WER = "WER: Test"
ORIGINAL_WER = "WER: Original Test"
HYPER = {"adapters": ["Adapter Dimensions", "Adapter Dropout", "Stochastic Depth", "Train Steps"], "finetuning": ["Train Steps", "Learning Rate"]}
CATEGORY = {"adapters": "Adapter Position", "finetuning": "Frozen Module"}


def original_scale(original_wer: float, baseline: float, max_degradation: float) -> float:
    return (max_degradation - min(max_degradation, abs(original_wer - baseline))) / max_degradation


def adapt_werr(adapted_wer: float, baseline: float) -> float:
    return max(baseline - adapted_wer, 0.0) / baseline


def add_scores(df: pd.DataFrame, dataset_col: str, baselines: Dict, max_degradation: float, test_col: str = TEST_WER, orig_col: str = ORIGINAL_WER) -> pd.DataFrame:
    missing = set(df[dataset_col].unique()) - set(baselines["adapted"])
    if missing:
        raise KeyError(f"no baseline WER for dataset groups {sorted(missing)}")
    df = df.copy()
    df["Original Scale"] = [original_scale(w, baselines["original"], max_degradation) for w in df[orig_col]]
    df["Adapt WERR"] = [adapt_werr(w, baselines["adapted"][g]) for w, g in zip(df[test_col], df[dataset_col])]
    df["Score"] = df["Original Scale"] * df["Adapt WERR"]
    return df.round({"Original Scale": 4, "Adapt WERR": 4, "Score": 4})


def rank(df: pd.DataFrame, exp_type: str, key: str, ascending: bool, test_col: str = TEST_WER, orig_col: str = ORIGINAL_WER) -> Dict[str, pd.DataFrame]:
    """Per category: hyper-parameter combinations with their means over dataset groups, best first."""
    hyper = [c for c in HYPER[exp_type] if c in df.columns]
    cols = list(dict.fromkeys([key, test_col, orig_col]))
    out = {}
    for cat in df[CATEGORY[exp_type]].unique():
        sub = df[df[CATEGORY[exp_type]] == cat]
        out[str(cat)] = sub.groupby(hyper, as_index=False)[cols].mean().sort_values(by=key, ascending=ascending).reset_index(drop=True)
    return out


def restrict(df: pd.DataFrame, fixed: Sequence[Tuple[str, str]]) -> pd.DataFrame:
    for name, value in fixed or []:
        col = df[name]
        df = df[col.astype(str) == str(value)] if col.dtype == object else df[col == type(col.iloc[0])(value)]
    return df


def report(title: str, ranked: Dict[str, pd.DataFrame], df: pd.DataFrame, exp_type: str, dataset_col: str, key: str, topk: int, show_analysis: bool) -> List[Dict]:
    hyper = [c for c in HYPER[exp_type] if c in df.columns]
    best = []
    print(f"\n{'#' * 8} {title} {'#' * 8}")
    for cat, table in ranked.items():
        print(f"\n== {cat.upper()} ==")
        if show_analysis:
            print(table.to_string(index=False))
        for k in range(min(topk, len(table))):
            row = table.iloc[k]
            print(f"-- top-{k + 1}: " + ", ".join(f"{h}={row[h]}" for h in hyper) + f"  |  mean {key} = {row[key]:.4f}")
            runs = df[df[CATEGORY[exp_type]].astype(str) == cat]
            for h in hyper:
                runs = runs[runs[h] == row[h]]
            for _, r in runs.sort_values(dataset_col).iterrows():
                print(f"     {r[dataset_col]:<28} {TEST_WER} {r[TEST_WER]:7.3f}   {ORIGINAL_WER} {r[ORIGINAL_WER]:7.3f}   Score {r['Score']:.4f}")
            if k == 0:
                best.append({"category": cat, "selection": title, **{h: row[h] for h in hyper}, key: float(row[key])})
    return best


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--csv", required=True)
    ap.add_argument("--dataset_type_column", required=True)
    ap.add_argument("--baselines", required=True, help="JSON with the un-adapted model's WER on the original domain and on every dataset group")
    ap.add_argument("--max_degradation", type=float, default=3.0)
    ap.add_argument("-ft", "--finetuning", action="store_true")
    ap.add_argument("--topk", type=int, default=1)
    ap.add_argument("--show_analysis", action="store_true")
    ap.add_argument("-uargs", "--unconstrained_args", nargs=2, action="append", default=[], metavar=("COLUMN", "VALUE"))
    ap.add_argument("-cargs", "--constrained_args", nargs=2, action="append", default=[], metavar=("COLUMN", "VALUE"))
    a = ap.parse_args(argv)
    exp_type = "finetuning" if a.finetuning else "adapters"
    with open(a.baselines) as f:
        baselines = json.load(f)
    df = pd.read_csv(a.csv)
    if exp_type == "finetuning" and CATEGORY[exp_type] in df:
        df[CATEGORY[exp_type]] = df[CATEGORY[exp_type]].replace("-", "null")
    df = add_scores(df, a.dataset_type_column, baselines, a.max_degradation)
    df.to_csv(a.csv, index=False)
    best = []
    un = restrict(df, a.unconstrained_args)
    best += report("unconstrained (lowest new-domain WER)", rank(un, exp_type, TEST_WER, True), un, exp_type, a.dataset_type_column, TEST_WER, a.topk, a.show_analysis)
    co = restrict(df, a.constrained_args)
    best += report("constrained (highest score)", rank(co, exp_type, "Score", False), co, exp_type, a.dataset_type_column, "Score", a.topk, a.show_analysis)
    return best


if __name__ == "__main__":
    main()
