"""RL prompts from JSONL files: codec, chat rendering, length filter, text rewards on decoded responses (CPU)."""
import json

from relax_b200.data.tokenizer import ByteCodec, PromptEncoder, build_codec, has_tokenizer_files
from relax_b200.rollout.data_source import JsonlPromptDataset, RolloutDataSource


def test_codec_roundtrip_and_prompt_encoder():
    c = ByteCodec(1024)
    ids = c.encode("héllo Answer: 42")
    assert c.decode(ids) == "héllo Answer: 42" and min(ids) >= 3
    assert c.decode([0, 1, 2, 900] + c.encode("ok")) == "ok"            # special / out-of-range ids decode to nothing
    plain = PromptEncoder(c, system_prompt="Be brief.")
    assert c.decode(plain("2+2?")) == "Be brief.\n2+2?"
    chat = PromptEncoder(c, apply_chat_template=True, system_prompt="Be brief.", max_prompt_len=200)
    text = c.decode(chat([{"role": "user", "content": [{"type": "image", "image": "x.png"}, {"type": "text", "text": "what?"}]}]))
    assert text.startswith("<|system|>\nBe brief.\n<|user|>\nwhat?\n") and text.endswith("<|assistant|>\n")
    assert chat("x" * 500) is None
    assert not has_tokenizer_files(None) and isinstance(build_codec(None, 512), ByteCodec)


def test_jsonl_dataset_filters_and_feeds_the_data_source(tmp_path):
    f1, f2 = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    f1.write_text(json.dumps({"q": "short one", "ans": 1, "meta": {"data_source": "gsm8k"}}) + "\n" + json.dumps({"q": "y" * 300, "ans": 2}) + "\n")
    f2.write_text(json.dumps({"q": "another", "ans": 3}) + "\n")
    enc = PromptEncoder(ByteCodec(1024), max_prompt_len=64)
    ds = JsonlPromptDataset(f"{f1},{f2}", enc, "q", "ans", "meta")
    assert len(ds) == 2 and ds.dropped == 1 and ds[0]["label"] == 1 and ds[0]["metadata"] == {"data_source": "gsm8k"}
    src = RolloutDataSource(ds, 2, shuffle=True, seed=1)
    groups = src.get_samples(3)                  # wraps into the second epoch
    assert len(groups) == 3 and all(len(g) == 2 for g in groups) and src.epoch == 1
    assert {g[0].label for g in groups} == {1, 3}


def test_colocated_loop_on_prompt_files_scores_decoded_text(tmp_path):
    from relax_b200.algo.loss import LossConfig
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"What is {i}+{i}?", "label": str(2 * i)}) for i in range(6)) + "\n")
    user = tmp_path / "rm.py"
    user.write_text("SEEN = []\ndef rm(sample):\n    SEEN.append((sample.prompt, sample.response, sample.label))\n    return float(len(sample.response) % 2)\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--prompt-data", str(f), "--input-key", "prompt",
                    "--label-key", "label", "--custom-rm-path", f"{user}:rm", "--rollout-shuffle"])
    c = Controller(a, device="cpu")
    m = c.runner.step()
    from relax_b200.rollout.custom_generate import load_object

    seen = load_object(f"{user}:SEEN")
    assert len(seen) == 4 and all(p.startswith("What is") and isinstance(r, str) and lab.isdigit() for p, r, lab in seen)
    assert 0.0 <= m["raw_reward_mean"] <= 1.0


def test_stop_strings_cut_the_response():
    from relax_b200.data.tokenizer import cut_at_stop_strings

    c = ByteCodec(1024)
    ids = c.encode("The answer is 42.</answer> and then more text")
    n = cut_at_stop_strings(c, ids, ["</answer>", "###"])
    assert c.decode(ids[:n]) == "The answer is 42.</answer>"
    assert cut_at_stop_strings(c, ids, ["nope"]) is None and cut_at_stop_strings(c, ids, []) is None
    assert cut_at_stop_strings(c, c.encode("###"), ["###"]) == 3


def test_rollout_stop_flag_trims_samples(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout.custom_generate import load_object

    user = tmp_path / "rm2.py"
    user.write_text("SEEN = []\ndef rm(sample):\n    SEEN.append((sample.response, sample.response_length, len(sample.rollout_log_probs)))\n    return 1.0\n")
    # random byte-level text: use a stop string that certainly occurs - every single byte value the model can emit
    stops = [chr(b) for b in range(32, 127)]
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "12", "--custom-rm-path", f"{user}:rm", "--rollout-stop"] + stops)
    c = Controller(a, device="cpu")
    c.runner.step()
    seen = load_object(f"{user}:SEEN")
    assert len(seen) == 4
    for text, n, nlp in seen:
        assert n == nlp and n <= 12
        if any(ch in text for ch in stops):                  # cut right after the first printable character
            assert sum(ch in stops for ch in text) == 1 and text[-1] in stops


def test_streaming_source_covers_epochs_and_resumes_exactly(tmp_path):
    from relax_b200.rollout.data_source import StreamingRolloutDataSource

    files = []
    for k in range(2):
        p = tmp_path / f"p{k}.jsonl"
        p.write_text("\n".join(json.dumps({"prompt": f"q{k}-{i}", "label": 10 * k + i}) for i in range(7)) + "\n")
        files.append(str(p))
    enc = PromptEncoder(ByteCodec(1024), max_prompt_len=64)
    mk = lambda: StreamingRolloutDataSource(",".join(files), enc, 1, buffer_size=4, seed=3)
    src = mk()
    first = [g[0].label for g in src.get_samples(14)]
    assert sorted(first) == sorted(list(range(7)) + list(range(10, 17))) and first != sorted(first)      # every row once, shuffled
    second = [g[0].label for g in src.get_samples(14)]
    assert sorted(second) == sorted(first) and second != first and src.epoch == 1                        # a new order per epoch
    a = mk()
    a.get_samples(5)
    st = a.state_dict()
    rest = [g[0].label for g in a.get_samples(12)]
    b = mk()
    b.load_state_dict(st)
    assert [g[0].label for g in b.get_samples(12)] == rest and b.group_index == a.group_index


def test_streaming_flag_in_the_loop(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller
    from relax_b200.rollout.data_source import StreamingRolloutDataSource

    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"What is {i}?", "label": str(i)}) for i in range(6)) + "\n")
    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--prompt-data", str(f), "--input-key", "prompt",
                    "--use-streaming-dataset", "--streaming-buffer-size", "3", "--rollout-shuffle"])
    c = Controller(a, device="cpu")
    assert isinstance(c.runner.data_source, StreamingRolloutDataSource)
    m = c.runner.step()
    assert m["response_tokens_local"] > 0


def test_resume_continues_the_prompt_stream(tmp_path):
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps({"prompt": f"What is {i}?", "label": str(i)}) for i in range(8)) + "\n")
    common = ["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
              "--rollout-max-response-len", "8", "--prompt-data", str(f), "--input-key", "prompt", "--label-key", "label",
              "--save", str(tmp_path / "ck"), "--load", str(tmp_path / "ck"), "--save-interval", "1"]
    c = Controller(parse_args(common + ["--num-rollout", "2"]), device="cpu")
    c.training_loop()
    assert c.runner.data_source.state_dict()["offset"] == 4
    c2 = Controller(parse_args(common + ["--num-rollout", "3"]), device="cpu")
    assert c2.start_rollout_id == 2 and c2.runner.data_source.state_dict()["offset"] == 4
    labels = [g[0].label for g in c2.runner.data_source.get_samples(2)]
    assert labels == ["4", "5"]


def test_tool_definitions_are_rendered_into_the_prompt(tmp_path):
    c = ByteCodec(4096)
    f = tmp_path / "t.jsonl"
    tools = [{"type": "function", "function": {"name": "search", "parameters": {}}}]
    f.write_text(json.dumps({"prompt": [{"role": "user", "content": "find it"}], "tools": json.dumps(tools)}) + "\n" +
                 json.dumps({"prompt": [{"role": "user", "content": "no tools"}]}) + "\n")
    ds = JsonlPromptDataset(str(f), PromptEncoder(c, apply_chat_template=True), "prompt", None, "metadata", tool_key="tools")
    with_tools, without = c.decode(ds[0]["prompt_tokens"]), c.decode(ds[1]["prompt_tokens"])
    assert with_tools.startswith("<|tools|>") and '"search"' in with_tools and "find it" in with_tools
    assert not without.startswith("<|tools|>") and ds[0]["label"] is None


def test_hf_codec_with_a_locally_built_tokenizer(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from relax_b200.data.tokenizer import HFCodec

    vocab = {"[UNK]": 0, "[EOS]": 1, "hello": 2, "world": 3, "what": 4, "is": 5, "?": 6, "user": 7, "assistant": 8}
    t = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    t.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=t, unk_token="[UNK]", eos_token="[EOS]")
    fast.chat_template = ("{% for m in messages %}{{ m['role'] }} {{ m['content'] }} {% endfor %}"
                          "{% if add_generation_prompt %}assistant {% endif %}")
    fast.save_pretrained(str(tmp_path))
    assert has_tokenizer_files(str(tmp_path))
    c = build_codec(str(tmp_path), 100)
    assert isinstance(c, HFCodec) and c.encode("hello world") == [2, 3] and c.decode([2, 3]) == "hello world" and c.eos_token_id == 1
    ids = PromptEncoder(c, apply_chat_template=True)([{"role": "user", "content": "what is hello ?"}])
    assert ids == [7, 4, 5, 2, 6, 8]
