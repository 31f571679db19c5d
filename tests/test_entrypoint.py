"""The train entrypoint end to end on CPU with the tiny model: colocated RL with save/resume, async mode, SFT."""
import json
import os

from relax_b200.checkpoint import dist_ckpt
from relax_b200.entrypoints.train import main

COMMON = ["--model-name", "tiny", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
          "--rollout-max-prompt-len", "8", "--rollout-max-response-len", "8", "--lr", "1e-4", "--max-tokens-per-gpu", "256"]


def test_colocated_run_saves_and_resumes(tmp_path):
    save = str(tmp_path / "ckpt")
    assert main(COMMON + ["--num-rollout", "2", "--save", save, "--save-interval", "1", "--colocate"]) == 0
    assert dist_ckpt.read_latest_iteration(save) == 1
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert [l["step"] for l in lines] == [0, 1] and "perf/step_time" in lines[0]
    # resume: starts at step 2, runs one more
    assert main(COMMON + ["--num-rollout", "3", "--save", save, "--load", save, "--save-interval", "1", "--colocate"]) == 0
    assert dist_ckpt.read_latest_iteration(save) == 2
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert [l["step"] for l in lines] == [0, 1, 2]


def test_fully_async_run(tmp_path):
    assert main(COMMON + ["--num-rollout", "3", "--fully-async", "--max-staleness", "1"]) == 0


def test_sft_run(tmp_path):
    data = tmp_path / "sft.jsonl"
    with open(data, "w") as f:
        for i in range(16):
            f.write(json.dumps({"prompt": f"say {i}", "response": f"number {i}"}) + "\n")
    save = str(tmp_path / "sft_ckpt")
    assert main(["--model-name", "tiny", "--loss-type", "sft_loss", "--prompt-data", str(data), "--num-rollout", "3",
                 "--global-batch-size", "4", "--lr", "1e-3", "--max-tokens-per-gpu", "512", "--save", save]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert len(lines) == 3 and lines[-1]["loss"] < lines[0]["loss"]


def test_model_shape_flags_follow_megatron_meaning():
    from relax_b200.config.arguments import model_config_from_args, parse_args

    shape = ["--colocate", "--num-layers", "2", "--hidden-size", "64", "--ffn-hidden-size", "128", "--num-attention-heads", "4",
             "--num-query-groups", "2", "--kv-channels", "16", "--vocab-size", "100"]
    c = model_config_from_args(parse_args(shape + ["--norm-epsilon", "1e-5", "--rotary-base", "500000", "--add-qkv-bias",
                                                   "--untie-embeddings-and-output-weights"]))
    assert (c.rms_norm_eps, c.rope_theta, c.qkv_bias, c.tie_word_embeddings, c.qk_layernorm) == (1e-5, 5e5, True, False, False)
    c = model_config_from_args(parse_args(shape + ["--qk-layernorm"]))
    assert c.qk_layernorm and c.tie_word_embeddings and not c.qkv_bias and c.rope_theta == 1e6
    # a preset keeps its own values unless a flag is given
    c = model_config_from_args(parse_args(["--colocate", "--model-name", "llama3-8b"]))
    assert c.rope_theta == 5e5 and c.rms_norm_eps == 1e-5 and not c.qk_layernorm
    c = model_config_from_args(parse_args(["--colocate", "--model-name", "llama3-8b", "--rotary-base", "1e6"]))
    assert c.rope_theta == 1e6


def test_engine_flags_reach_the_rollout_engine():
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--sglang-page-size", "8", "--sglang-max-running-requests", "3",
                    "--sglang-chunked-prefill-size", "64", "--sglang-disable-cuda-graph"])
    eng = Controller(a, device="cpu").runner.engine
    assert eng.block_size == 8 and eng.max_running == 3 and eng.max_prefill_tokens == 64 and not eng.use_cuda_graph


def test_standalone_services_start_and_answer(tmp_path):
    import json
    import re
    import subprocess
    import sys
    import time
    import urllib.request

    from relax_b200.utils.visualize import dump_rollout
    from relax_b200.types import Sample

    dump_rollout(str(tmp_path), 0, [Sample(response="x", response_length=1, reward=1.0, tokens=[1, 2])])
    for svc, extra, path in (("viewer", ["--dir", str(tmp_path)], "/api/steps"), ("coordinator", [], "/health"),
                             ("metrics", ["--dir", str(tmp_path)], None)):
        p = subprocess.Popen([sys.executable, "-m", "relax_b200.entrypoints.serve", svc, "--max-seconds", "20"] + extra,
                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        try:
            line = p.stdout.readline()
            m = re.search(r"listening on (http://[\d.]+:\d+)", line)
            assert m, line
            if path:
                body = urllib.request.urlopen(m.group(1) + path, timeout=10).read()
                assert body
            else:
                req = urllib.request.Request(m.group(1) + "/log_metric", data=json.dumps({"step": 1, "name": "loss", "value": 0.5}).encode(),
                                             headers={"Content-Type": "application/json"})
                assert urllib.request.urlopen(req, timeout=10).status == 200
        finally:
            p.terminate()
            p.wait(10)


def test_openapi_routes_exist_on_live_servers(tmp_path):
    import json
    import urllib.error
    import urllib.request

    from relax_b200.metrics.service import MetricsService, serve as serve_metrics
    from relax_b200.utils import openapi
    from relax_b200.weight_sync.dcs import Coordinator, serve as serve_coord

    assert openapi.main(["--service", "all", "--out-dir", str(tmp_path)]) == 0
    spec = json.load(open(tmp_path / "coordinator.openapi.json"))
    assert "/recv_weight_meta" in spec["paths"] and spec["openapi"].startswith("3.")
    for name, (srv, url) in (("metrics", serve_metrics(MetricsService([]))), ("coordinator", serve_coord(Coordinator()))):
        try:
            for method, path, _, schema in openapi.ROUTES[name]:
                if path == "/recv_weight_meta":
                    continue            # a long poll: it answers only once a layout is published
                data = json.dumps({}).encode() if method == "post" else None
                req = urllib.request.Request(url + path, data=data, headers={"Content-Type": "application/json"}, method=method.upper())
                try:
                    code = urllib.request.urlopen(req, timeout=10).status
                except urllib.error.HTTPError as e:
                    code = e.code
                assert code != 404, (name, path)       # the route exists (an empty body may be a 400)
        finally:
            srv.shutdown()
            srv.server_close()


def test_timeline_dump(tmp_path):
    import json
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    a = parse_args(["--model-name", "tiny", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2", "--global-batch-size", "4",
                    "--num-rollout", "1", "--rollout-max-response-len", "8", "--timeline-dump-dir", str(tmp_path / "tl")])
    Controller(a, device="cpu").training_loop()
    tr = json.load(open(tmp_path / "tl" / "timeline_rank0.json"))
    names = {e["name"] for e in (tr["traceEvents"] if isinstance(tr, dict) else tr)}
    assert {"rollout", "train"} <= names


def test_openapi_chat_routes_exist_on_a_live_server():
    import json
    import urllib.error
    import urllib.request

    from relax_b200.rollout.agentic import Tokenizer
    from relax_b200.rollout.openai_api import ChatService, serve
    from relax_b200.utils import openapi

    tok = Tokenizer(encode=lambda s: [ord(c) for c in s], decode=lambda t: "".join(chr(97 + x % 26) for x in t))
    gen = lambda prompts, n, keys: [([5, 6], [-0.1, -0.2], "stop", [0]) for _ in prompts]
    srv, url = serve(ChatService(gen, tok))
    try:
        for method, path, _, schema in openapi.ROUTES["chat"]:
            body = {"messages": [{"role": "user", "content": "hi"}]} if method == "post" else None
            req = urllib.request.Request(url + path, data=json.dumps(body).encode() if body else None,
                                         headers={"Content-Type": "application/json"}, method=method.upper())
            assert urllib.request.urlopen(req, timeout=10).status == 200, path
    finally:
        srv.shutdown()
        srv.server_close()


def test_reference_from_a_training_checkpoint_step(tmp_path):
    """``--ref-load <checkpoint dir> --ref-ckpt-step N``: the frozen reference is the policy saved at iteration N of
    another run, not the current initialisation."""
    import torch

    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    save = str(tmp_path / "ckpt")
    assert main(COMMON + ["--num-rollout", "2", "--save", save, "--save-interval", "1", "--colocate", "--lr", "1e-2"]) == 0
    a = parse_args(COMMON + ["--num-rollout", "1", "--colocate", "--ref-load", save, "--ref-ckpt-step", "0", "--kl-loss-coef", "0.01",
                             "--use-kl-loss"])
    c = Controller(a, device="cpu")
    c._maybe_resume()
    actor = c.runner.actor
    saved = dist_ckpt.load_full_tensors(dist_ckpt.iter_dir(save, 0))
    name, p = next((n, p) for n, p in actor.model.named_parameters() if n.endswith("linear_proj.weight"))
    actor.switch_model("ref")
    assert torch.allclose(p.detach(), saved[name].to(p.dtype))
    actor.switch_model("actor")
    assert not torch.allclose(p.detach(), saved[name].to(p.dtype)), "the policy itself keeps its own initialisation"
    c.runner.close()


def test_sequence_classification_runs(tmp_path):
    """``--loss-type seq_cls_loss --num-labels N`` fine-tunes the class head; single- and multi-label."""
    data = tmp_path / "cls.jsonl"
    with open(data, "w") as f:
        for i in range(16):
            f.write(json.dumps({"prompt": "aaaa" if i % 2 else "zzzz zzzz", "label": i % 2, "labels": [i % 2, 2] if i % 2 else [0]}) + "\n")
    base = ["--model-name", "tiny", "--prompt-data", str(data), "--global-batch-size", "8", "--num-rollout", "8", "--lr", "1e-3",
            "--max-tokens-per-gpu", "256", "--loss-type", "seq_cls_loss"]
    save = str(tmp_path / "a")
    assert main(base + ["--num-labels", "2", "--save", save]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    get = lambda l, k: l.get("train/" + k, l.get(k))
    assert get(lines[-1], "accuracy") >= get(lines[0], "accuracy") and get(lines[-1], "loss") < get(lines[0], "loss")
    assert lines[0]["total_tokens_local"] > 8
    save = str(tmp_path / "b")
    assert main(base + ["--num-labels", "3", "--problem-type", "multi_label_classification", "--label-key", "labels", "--save", save]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert get(lines[-1], "label_accuracy") is not None and get(lines[-1], "loss") < get(lines[0], "loss")


def test_vision_language_run_through_the_entrypoint(tmp_path):
    """A vision-language preset through the train entrypoint: synthetic image prompts, tower frozen by the switch."""
    save = str(tmp_path / "vl")
    assert main(["--model-name", "tiny-vl", "--colocate", "--rollout-batch-size", "2", "--n-samples-per-prompt", "2",
                 "--global-batch-size", "4", "--rollout-max-prompt-len", "24", "--rollout-max-response-len", "8", "--lr", "1e-4",
                 "--max-tokens-per-gpu", "512", "--num-rollout", "2", "--freeze-vision-model", "--save", save]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert len(lines) == 2 and lines[-1]["train_rollout_logprob_abs_diff"] < 1e-3
    assert lines[-1]["rollout/prompt_lengths"] == 24         # text + image placeholders


def test_sft_with_a_periodic_predict_pass(tmp_path):
    """``--sft-predict-interval``: every second step the current weights answer the evaluation conversations (cut before
    their last assistant turn) and the completions land in <save>/predict/."""
    data = tmp_path / "sft.jsonl"
    with open(data, "w") as f:
        for i in range(16):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"say {i}"}, {"role": "assistant", "content": f"number {i}"}]}) + "\n")
    save = str(tmp_path / "sft_ckpt")
    assert main(["--model-name", "tiny", "--loss-type", "sft_loss", "--prompt-data", str(data), "--num-rollout", "4",
                 "--global-batch-size", "4", "--lr", "1e-3", "--max-tokens-per-gpu", "512", "--save", save,
                 "--sft-predict-interval", "2", "--eval-size", "3", "--rollout-max-response-len", "6"]) == 0
    files = sorted(os.listdir(os.path.join(save, "predict")))
    assert files == ["predictions_step_2.jsonl", "predictions_step_4.jsonl"]
    rows = [json.loads(l) for l in open(os.path.join(save, "predict", files[0]))]
    assert len(rows) == 3 and all(r["prompt"][0]["role"] == "user" and r["reference"].startswith("number ") for r in rows)
    assert all(isinstance(r["prediction"], str) and r["finish_reason"] in ("length", "stop") for r in rows)
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    assert [("predict/samples" in l) for l in lines] == [False, True, False, True]


def test_sft_periodic_evaluation_ppl_and_classification(tmp_path):
    """``--eval-interval`` under SFT: held-out perplexity for the language-model loss, accuracy / macro-F1 for the class head."""
    data = tmp_path / "sft.jsonl"
    with open(data, "w") as f:
        for i in range(16):
            f.write(json.dumps({"prompt": f"say {i % 4}", "response": f"number {i % 4}"}) + "\n")
    save = str(tmp_path / "sft_ckpt")
    assert main(["--model-name", "tiny", "--loss-type", "sft_loss", "--prompt-data", str(data), "--num-rollout", "6",
                 "--global-batch-size", "8", "--lr", "3e-3", "--max-tokens-per-gpu", "512", "--save", save,
                 "--eval-interval", "3", "--eval-size", "4"]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save, "metrics.jsonl"))]
    ev = [l for l in lines if "eval/ppl" in l]
    assert [l["step"] for l in ev] == [2, 5] and ev[1]["eval/nll"] < ev[0]["eval/nll"] and ev[0]["eval/tokens"] > 0
    cls = tmp_path / "cls.jsonl"
    with open(cls, "w") as f:
        for i in range(24):
            f.write(json.dumps({"text": "good " * (1 + i % 3) if i % 2 else "bad " * (1 + i % 3), "label": i % 2}) + "\n")
    save2 = str(tmp_path / "cls_ckpt")
    assert main(["--model-name", "tiny", "--loss-type", "seq_cls_loss", "--num-labels", "2", "--prompt-data", str(cls), "--input-key", "text",
                 "--num-rollout", "8", "--global-batch-size", "8", "--lr", "3e-3", "--max-tokens-per-gpu", "512", "--save", save2,
                 "--eval-interval", "4", "--eval-size", "8"]) == 0
    lines = [json.loads(l) for l in open(os.path.join(save2, "metrics.jsonl"))]
    ev = [l for l in lines if "eval/accuracy" in l]
    assert len(ev) == 2 and ev[-1]["eval/samples"] == 8 and ev[-1]["eval/accuracy"] >= 0.75 and 0 <= ev[-1]["eval/macro_f1"] <= 1


def test_sft_resume_continues_the_data_stream(tmp_path):
    """The SFT data cursor travels with the checkpoint: a resumed run trains on the samples that follow the last trained
    batch (not on what the prefetcher had already read, and not from the top of the file)."""
    from relax_b200.config.arguments import parse_args
    from relax_b200.orchestration.controller import Controller

    data = tmp_path / "sft.jsonl"
    with open(data, "w") as f:
        for i in range(40):
            f.write(json.dumps({"prompt": f"q{i}", "response": f"a{i}"}) + "\n")
    save = str(tmp_path / "ck")
    base = ["--model-name", "tiny", "--loss-type", "sft_loss", "--prompt-data", str(data), "--global-batch-size", "4", "--lr", "1e-3",
            "--max-tokens-per-gpu", "512", "--save", save, "--save-interval", "1", "--sft-prefetch-buffer-size", "16"]
    assert main(base + ["--num-rollout", "3"]) == 0
    it = dist_ckpt.read_latest_iteration(save)
    st = json.load(open(os.path.join(dist_ckpt.iter_dir(save, it), "rollout_data_source.json")))
    assert st["line"] == 12 and st["file_index"] == 0                 # three batches of four samples were trained on
    c = Controller(parse_args(base + ["--num-rollout", "5", "--load", save]), device="cpu")
    assert c.runner.state_dict()["line"] == 12
    nxt = next(c.runner.batches)
    from relax_b200.data.tokenizer import ByteCodec

    text = ByteCodec(c.model_cfg.vocab_size).decode(nxt["tokens"][0])
    assert "q12" in text and "a12" in text
