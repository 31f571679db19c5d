"""Dataset preparation commands: turn raw benchmark / chat files into the JSONL rows the prompt loader reads
(``{"prompt": [messages], "label": ..., "metadata": {...}}``).

Covers the reference's dataset tools (scripts/tools/process_aime.py, process_openr1.py, process_avqa.py,
process_nextqa.py, process_tool_chat.py): an instruction prefix for math evaluation sets, multimodal question
rows with media placeholders, and flattened tool-call logs rebuilt into chat messages with structured
``tool_calls``.

    python -m relax_b200.data.preprocess aime --input aime.jsonl --output aime.prompts.jsonl
    python -m relax_b200.data.preprocess tool_chat --input raw.jsonl --output chat.jsonl
    python -m relax_b200.data.preprocess mmqa --input openr1.jsonl --output openr1.prompts.jsonl --media-key image
"""
from __future__ import annotations

import argparse
import json
from typing import Any, Dict, Iterable, Iterator, List, Optional

MATH_INSTRUCTION = ("Solve the following math problem step by step. The last line of your response should be of the "
                    "form Answer: \\boxed{$Answer} where $Answer is the answer to the problem.\n\n")
MM_INSTRUCTION = ("First output the thinking process in <think> </think> tags and then output the final answer in "
                  "<answer> </answer> tags.")


def read_jsonl(path: str) -> Iterator[dict]:
    with open(path, encoding="utf-8") as f:
        for line in f:
            if line.strip():
                yield json.loads(line)


def write_jsonl(path: str, rows: Iterable[dict]) -> int:
    n = 0
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
            n += 1
    return n


def _as_messages(prompt) -> List[dict]:
    if isinstance(prompt, str):
        return [{"role": "user", "content": prompt}]
    return [dict(m) for m in prompt]


def math_eval_row(item: dict, prefix: str = MATH_INSTRUCTION) -> dict:
    """Prepend the answer-format instruction to the first user turn (idempotent)."""
    msgs = _as_messages(item.get("prompt", item.get("question", item.get("problem", ""))))
    first = next((m for m in msgs if m.get("role") == "user"), msgs[0])
    if not str(first["content"]).startswith(prefix):
        first["content"] = prefix + str(first["content"])
    label = item.get("label", item.get("answer", item.get("solution")))
    out = {"prompt": msgs, "label": label}
    if "metadata" in item:
        out["metadata"] = item["metadata"]
    return out


def multimodal_qa_row(item: dict, media_key: str = "image", question_key: str = "problem", answer_key: str = "solution",
                      options_key: Optional[str] = None, data_source: str = "") -> dict:
    """One question about one or several media items -> a user turn whose content lists the media parts first and
    the text last (the layout :func:`relax_b200.data.multimodal.process_multimodal_info` scans)."""
    media = item.get(media_key)
    media = media if isinstance(media, list) else ([media] if media is not None else [])
    text = str(item.get(question_key, ""))
    if options_key and item.get(options_key):
        text += "\n" + "\n".join(f"{chr(65 + i)}. {o}" for i, o in enumerate(item[options_key]))
    parts: List[dict] = [{"type": media_key, media_key: m} for m in media]
    parts.append({"type": "text", "text": f"{text}\n{MM_INSTRUCTION}"})
    ans = item.get(answer_key)
    if isinstance(ans, int) and options_key:
        ans = chr(65 + ans)
    return {"prompt": [{"role": "user", "content": parts}], "label": ans,
            "metadata": {"data_source": data_source or item.get("data_source", ""), "num_media": len(media)}}


def _tool_call_from_text(content: str) -> Dict[str, Any]:
    obj = json.loads(content)
    args = obj.get("arguments", obj.get("parameters", {}))
    if isinstance(args, str):
        try:
            args = json.loads(args)
        except ValueError:
            pass
    return {"type": "function", "function": {"name": obj["name"], "arguments": args}}


def tool_chat_row(record: dict) -> dict:
    """Flattened tool-call logs -> chat messages: ``tools`` parsed from its JSON string; a ``tool_call`` turn becomes
    an assistant message with ``tool_calls`` (consecutive ones are merged into one assistant turn); a
    ``tool_response`` turn becomes a ``tool`` message."""
    tools = record.get("tools")
    if isinstance(tools, str):
        tools = json.loads(tools) if tools.strip() else []
    out: List[dict] = []
    for m in record["messages"]:
        role, content = m.get("role"), m.get("content", "")
        if role == "tool_call":
            call = _tool_call_from_text(content)
            if out and out[-1]["role"] == "assistant" and out[-1].get("tool_calls") and not out[-1].get("_closed"):
                out[-1]["tool_calls"].append(call)
            else:
                out.append({"role": "assistant", "content": "", "tool_calls": [call]})
        elif role == "tool_response":
            if out and out[-1]["role"] == "assistant":
                out[-1]["_closed"] = True
            out.append({"role": "tool", "content": content})
        else:
            out.append({"role": role, "content": content})
    for m in out:
        m.pop("_closed", None)
    return {**{k: v for k, v in record.items() if k not in ("tools", "messages")}, "tools": tools or [], "messages": out}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("aime", "tool_chat", "mmqa"):
        sp = sub.add_parser(name)
        sp.add_argument("--input", required=True)
        sp.add_argument("--output", default=None, help="default: rewrite the input file")
    mm = sub.choices["mmqa"]
    mm.add_argument("--media-key", default="image")
    mm.add_argument("--question-key", default="problem")
    mm.add_argument("--answer-key", default="solution")
    mm.add_argument("--options-key", default=None)
    mm.add_argument("--data-source", default="")
    a = ap.parse_args(argv)
    rows = list(read_jsonl(a.input))
    if a.cmd == "aime":
        out = [math_eval_row(r) for r in rows]
    elif a.cmd == "tool_chat":
        out = [tool_chat_row(r) for r in rows]
    else:
        out = [multimodal_qa_row(r, a.media_key, a.question_key, a.answer_key, a.options_key, a.data_source) for r in rows]
    n = write_jsonl(a.output or a.input, out)
    print(f"{a.cmd}: wrote {n} rows to {a.output or a.input}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
