"""Dataset preparation commands (CPU)."""
import json

from relax_b200.data import preprocess as P


def test_math_prefix_is_idempotent(tmp_path):
    f = tmp_path / "aime.jsonl"
    f.write_text(json.dumps({"prompt": [{"role": "user", "content": "What is 2+2?"}], "label": "4"}) + "\n" +
                 json.dumps({"problem": "1+1?", "answer": 2}) + "\n")
    assert P.main(["aime", "--input", str(f)]) == 0
    assert P.main(["aime", "--input", str(f)]) == 0            # a second pass changes nothing
    rows = list(P.read_jsonl(str(f)))
    assert rows[0]["prompt"][0]["content"].count("Solve the following") == 1 and rows[0]["label"] == "4"
    assert rows[1]["prompt"][0]["content"].endswith("1+1?") and rows[1]["label"] == 2


def test_tool_chat_conversion():
    rec = {"id": 7, "tools": json.dumps([{"name": "search", "parameters": {}}]),
           "messages": [{"role": "user", "content": "find x"},
                        {"role": "tool_call", "content": json.dumps({"name": "search", "arguments": "{\"q\": \"x\"}"})},
                        {"role": "tool_call", "content": json.dumps({"name": "open", "arguments": {"id": 1}})},
                        {"role": "tool_response", "content": "result"},
                        {"role": "tool_call", "content": json.dumps({"name": "search", "arguments": {"q": "y"}})},
                        {"role": "tool_response", "content": "r2"},
                        {"role": "assistant", "content": "done"}]}
    out = P.tool_chat_row(rec)
    roles = [m["role"] for m in out["messages"]]
    assert roles == ["user", "assistant", "tool", "assistant", "tool", "assistant"] and out["id"] == 7
    calls = out["messages"][1]["tool_calls"]
    assert [c["function"]["name"] for c in calls] == ["search", "open"] and calls[0]["function"]["arguments"] == {"q": "x"}
    assert isinstance(out["tools"], list) and out["tools"][0]["name"] == "search"
    assert all("_closed" not in m for m in out["messages"])


def test_multimodal_rows_feed_the_preprocessor(tmp_path):
    import numpy as np

    from relax_b200.data.multimodal import extract_vision_info

    row = P.multimodal_qa_row({"image": ["a.png", "b.png"], "problem": "Which is larger?", "options": ["left", "right"], "solution": 1},
                              options_key="options", data_source="openr1mm")
    parts = row["prompt"][0]["content"]
    assert [p["type"] for p in parts] == ["image", "image", "text"] and "B. right" in parts[-1]["text"] and row["label"] == "B"
    assert row["metadata"] == {"data_source": "openr1mm", "num_media": 2} and len(extract_vision_info(row["prompt"])) == 2
    f = tmp_path / "in.jsonl"
    f.write_text(json.dumps({"video": "clip.npy", "q": "what happens", "a": "it rains"}) + "\n")
    out = tmp_path / "out.jsonl"
    P.main(["mmqa", "--input", str(f), "--output", str(out), "--media-key", "video", "--question-key", "q", "--answer-key", "a"])
    r = next(P.read_jsonl(str(out)))
    assert r["prompt"][0]["content"][0] == {"type": "video", "video": "clip.npy"} and r["label"] == "it rains"
