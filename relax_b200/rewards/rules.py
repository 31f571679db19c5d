"""Rule-based scorers registered under the reference's ``--rm-type`` names
(relax/engine/rewards/: deepscaler, dapo/math, f1, gpqa, multiple_choice,
geo3k, openr1mm) plus the synthetic ``parity`` reward of the benchmarks."""
from __future__ import annotations

import re
import string
from collections import Counter
from typing import Optional

from . import register_reward

# --------------------------------------------------------------------------- synthetic


@register_reward("parity", note="1 if the response's token count is even else 0")
def parity_reward(sample) -> float:
    return 1.0 if sample.response_length % 2 == 0 else 0.0


@register_reward("token_sum_parity", note="1 if the sum of response token ids is even")
def token_sum_parity_reward(sample) -> float:
    resp = sample.tokens[len(sample.tokens) - sample.response_length:]
    return 1.0 if sum(resp) % 2 == 0 else 0.0


@register_reward("random", note="deterministic pseudo-random reward from the sample index")
def random_reward(sample) -> float:
    return float((1103515245 * (int(sample.index or 0) + 12345)) % 1000) / 1000.0


# --------------------------------------------------------------------------- math


def last_boxed_only_string(s: str) -> Optional[str]:
    i = s.rfind("\\boxed")
    if i < 0:
        i = s.rfind("\\fbox")
        if i < 0:
            return None
    depth, j, start = 0, i, None
    while j < len(s):
        if s[j] == "{":
            depth += 1
            if start is None:
                start = j
        elif s[j] == "}":
            depth -= 1
            if depth == 0 and start is not None:
                return s[i:j + 1]
        j += 1
    return None


def remove_boxed(s: str) -> str:
    m = re.match(r"\\(?:boxed|fbox)\s*\{(.*)\}$", s, flags=re.S)
    return m.group(1) if m else s


def _strip_math(s: str) -> str:
    s = s.strip().replace("\n", "").replace("\\!", "").replace("\\ ", "").replace(" ", "")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*([^}]*)\}", r"\1", s)
    s = s.replace("\\%", "").replace("%", "")
    if s.startswith("0.") is False and s.startswith("."):
        s = "0" + s
    s = re.sub(r"^[a-zA-Z]\s*=", "", s)
    s = s.rstrip(".")
    m = re.fullmatch(r"\\frac(\d)(\d)", s)
    if m:
        s = f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}"
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    if m:
        s = f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}"
    if re.fullmatch(r"-?\d+\.0+", s):
        s = s.split(".")[0]
    return s.replace(",", "") if re.fullmatch(r"-?[\d,]+(\.\d+)?", s) else s


def _to_float(s: str) -> Optional[float]:
    m = re.fullmatch(r"\\frac\{(-?\d+)\}\{(\d+)\}", s)
    if m and int(m.group(2)) != 0:
        return int(m.group(1)) / int(m.group(2))
    try:
        return float(s)
    except ValueError:
        return None


def math_equal(pred: str, truth: str) -> bool:
    a, b = _strip_math(pred), _strip_math(truth)
    if a == b:
        return True
    fa, fb = _to_float(a), _to_float(b)
    return fa is not None and fb is not None and abs(fa - fb) <= 1e-6 * max(1.0, abs(fb))


def extract_answer(response: str) -> Optional[str]:
    b = last_boxed_only_string(response)
    if b is not None:
        return remove_boxed(b)
    m = re.findall(r"(?i)answer\s*[:：]\s*([^\n]+)", response)
    return m[-1].strip() if m else None


@register_reward("deepscaler", note="answer after </think> must match label; 0/1")
def deepscaler_reward(sample) -> float:
    resp = sample.response
    if "</think>" in resp:
        resp = resp.split("</think>")[-1]
    elif "<think>" in resp:
        return 0.0
    ans = extract_answer(resp)
    if ans is None or sample.label is None:
        return 0.0
    labels = sample.label if isinstance(sample.label, (list, tuple)) else [sample.label]
    return 1.0 if any(math_equal(ans, str(remove_boxed(l) if "\\boxed" in str(l) else l)) for l in labels) else 0.0


@register_reward("math", note="boxed answer equals label; 0/1")
def math_reward(sample) -> float:
    ans = extract_answer(sample.response)
    return 1.0 if ans is not None and sample.label is not None and math_equal(ans, str(sample.label)) else 0.0


@register_reward("dapo", note="+1 correct / -1 wrong, last 300 chars, 'Answer:' format")
def dapo_reward(sample) -> dict:
    tail = sample.response[-300:]
    m = re.findall(r"(?i)Answer\s*:\s*([^\n]+)", tail)
    pred = m[-1].strip() if m else None
    if pred is None:
        b = last_boxed_only_string(tail)
        pred = remove_boxed(b) if b else None
    ok = pred is not None and sample.label is not None and math_equal(pred, str(sample.label))
    return {"score": 1.0 if ok else -1.0, "acc": bool(ok), "pred": pred}


# --------------------------------------------------------------------------- QA


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def f1_score(pred: str, truth: str) -> float:
    p, t = normalize_answer(pred).split(), normalize_answer(truth).split()
    if not p or not t:
        return float(p == t)
    common = Counter(p) & Counter(t)
    n = sum(common.values())
    if n == 0:
        return 0.0
    pr, rc = n / len(p), n / len(t)
    return 2 * pr * rc / (pr + rc)


@register_reward("f1")
def f1_reward(sample) -> float:
    labels = sample.label if isinstance(sample.label, (list, tuple)) else [sample.label]
    return max(f1_score(sample.response, str(l)) for l in labels)


def _choice_letter(resp: str) -> Optional[str]:
    resp = resp.split("</think>")[-1]
    for pat in (r"(?i)answer\s*(?:is|:)?\s*\(?([A-J])\)?\b", r"\\boxed\{\(?([A-J])\)?\}", r"\b([A-J])\b(?!.*\b[A-J]\b)"):
        m = re.findall(pat, resp, flags=re.S)
        if m:
            return m[-1].upper()
    return None


@register_reward("multiple_choice")
def multiple_choice_reward(sample) -> float:
    return 1.0 if _choice_letter(sample.response) == str(sample.label).strip().upper() else 0.0


register_reward("gpqa", multiple_choice_reward, note="letter match after stripping chain of thought")


@register_reward("geo3k", note="0.9 * accuracy + 0.1 * <think>..</think>\\boxed{} format")
def geo3k_reward(sample) -> float:
    fmt = 1.0 if re.fullmatch(r"<think>.*</think>.*\\boxed\{.*\}.*", sample.response, flags=re.S) else 0.0
    ans = extract_answer(sample.response)
    acc = 1.0 if ans is not None and math_equal(ans, str(sample.label)) else 0.0
    return 0.9 * acc + 0.1 * fmt


@register_reward("openr1mm", note="accuracy + format on <think>/<answer> tags")
def openr1mm_reward(sample) -> float:
    m = re.search(r"<answer>(.*?)</answer>", sample.response, flags=re.S)
    fmt = 1.0 if re.fullmatch(r"\s*<think>.*?</think>\s*<answer>.*?</answer>\s*", sample.response, flags=re.S) else 0.0
    acc = 1.0 if m and math_equal(m.group(1), str(sample.label)) else 0.0
    return acc + fmt


# --------------------------------------------------------------------------- instruction following (ifbench style)
def _count_words(s: str) -> int:
    return len(re.findall(r"\b\w+\b", s))


_IF_CHECKS = {
    "min_words": lambda r, v: _count_words(r) >= int(v),
    "max_words": lambda r, v: _count_words(r) <= int(v),
    "min_sentences": lambda r, v: len([x for x in re.split(r"[.!?]+", r) if x.strip()]) >= int(v),
    "include_keywords": lambda r, v: all(k.lower() in r.lower() for k in v),
    "forbidden_words": lambda r, v: not any(re.search(rf"\b{re.escape(k)}\b", r, flags=re.I) for k in v),
    "num_paragraphs": lambda r, v: len([p for p in re.split(r"\n\s*\n", r.strip()) if p.strip()]) == int(v),
    "num_bullets": lambda r, v: len(re.findall(r"^\s*[\*\-] ", r, flags=re.M)) == int(v),
    "all_lowercase": lambda r, v: (r == r.lower()) == bool(v),
    "all_uppercase": lambda r, v: (r == r.upper()) == bool(v),
    "ends_with": lambda r, v: r.strip().endswith(str(v)),
    "starts_with": lambda r, v: r.strip().startswith(str(v)),
    "json_format": lambda r, v: _is_json(r) == bool(v),
    "no_commas": lambda r, v: ("," not in r) == bool(v),
}


def _is_json(r: str) -> bool:
    import json

    s = r.strip()
    s = re.sub(r"^```(?:json)?|```$", "", s.strip(), flags=re.M).strip()
    try:
        json.loads(s)
        return True
    except ValueError:
        return False


@register_reward("ifbench", note="fraction of the label's verifiable constraints the response satisfies")
def ifbench_reward(sample) -> float:
    """``sample.label``: dict (or JSON string) constraint -> argument, e.g. ``{"min_words": 50, "forbidden_words": ["very"]}``.
    Unknown constraints count as failed, so a typo in the data shows up as a low score instead of a free point."""
    import json

    spec = sample.label
    if isinstance(spec, str):
        try:
            spec = json.loads(spec)
        except ValueError:
            return 0.0
    if not isinstance(spec, dict) or not spec:
        return 0.0
    resp = sample.response.split("</think>")[-1]
    ok = 0
    for k, v in spec.items():
        fn = _IF_CHECKS.get(k)
        try:
            ok += 1 if fn is not None and fn(resp, v) else 0
        except (TypeError, ValueError):
            pass
    return ok / len(spec)


# --------------------------------------------------------------------------- remote / generative judges
@register_reward("remote_rm", note="POST {prompt, response, label} to --rm-url and read 'reward' from the JSON reply")
def remote_rm_reward(sample, url: Optional[str] = None, timeout: float = 30.0) -> float:
    import json
    import os
    import urllib.request

    url = url or os.environ.get("RELAX_RM_URL")
    if not url:
        raise ValueError("remote_rm needs a reward-model URL (--rm-url / RELAX_RM_URL)")
    body = json.dumps({"prompt": str(sample.prompt), "response": sample.response, "label": sample.label}).encode()
    req = urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        out = json.loads(r.read())
    return float(out["reward"] if isinstance(out, dict) else out)


# --------------------------------------------------------------------------- mixed-source routing
_STOP_MARKS = ("<|im_end|>", "<|endoftext|>", "</s>")


def _cut_at_stop(text: str) -> str:
    cut = [i for i in (text.find(m) for m in _STOP_MARKS) if i > 0]
    return text[:min(cut)] if cut else text


def _leading_number(s: str) -> Optional[float]:
    m = re.match(r"^\s*\$?\s*(-?\d[\d,]*(?:\.\d+)?)", s)
    return float(m.group(1).replace(",", "")) if m else None


@register_reward("gsm8k", note="+1 / -1; 'Answer: x' or '#### x'; text after an end-of-sequence marker ignored; more than five '####' = -1")
def gsm8k_reward(sample) -> float:
    """Grade-school-math scorer hardened against two failure modes of small policies: text emitted after a stop
    marker, and reward hacking by repeating the answer separator.  A prediction with a unit suffix ("100 miles")
    counts when its leading number equals the label."""
    label = sample.label
    if isinstance(label, dict):
        label = label.get("ground_truth") or label.get("answer", "")
    resp = _cut_at_stop(sample.response)
    if resp.count("####") > 5:
        return -1.0
    tail = resp[-300:]
    found = re.findall(r"(?i)answer\s*:\s*([^\n]+)", tail) or re.findall(r"####\s*(\$?-?[\d,]+(?:\.\d+)?)", tail)
    if not found:
        return -1.0
    pred = found[-1].strip()
    if math_equal(pred, str(label)):
        return 1.0
    a, b = _leading_number(pred), _to_float(_strip_math(str(label)))
    return 1.0 if a is not None and b is not None and abs(a - b) < 1e-9 else -1.0


@register_reward("mopd", note="routes by metadata['data_source']: geo3k -> math 0/1, openr1mm, dapo -> its scalar score, else gsm8k")
def mopd_reward(sample) -> float:
    """One scalar per sample for multi-source on-policy distillation data: every source is scored exactly as its own
    ``rm_type`` would score it (relax/engine/rewards/mopd.py get_mopd_reward)."""
    src = str((sample.metadata or {}).get("data_source", "")).lower()
    if "geometry3k" in src or "geo3k" in src:
        return math_reward(sample)
    if "multimodal-open-r1" in src or "openr1mm" in src:
        return float(openr1mm_reward(sample))
    if "dapo" in src:
        return float(dapo_reward(sample)["score"])
    return gsm8k_reward(sample)


def make_dapo_genrm_reward(genrm):
    """DAPO scoring with a generative judge for the answers the rule cannot parse: rule says correct -> +1; rule finds
    an answer and it is wrong -> -1; no parsable answer -> ask the generative grader (``relax_b200.rewards.genrm.GenRM``)."""
    def fn(sample) -> dict:
        base = dapo_reward(sample)
        if base.get("pred") not in (None, "", "[INVALID]"):
            return base
        score = genrm.score([str(sample.prompt)], [str(sample.label)], [sample.response])[0]
        return {"score": 1.0 if score >= 0.5 else -1.0, "acc": score >= 0.5, "pred": "[GENRM]"}

    return fn
