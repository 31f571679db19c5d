"""A minimal agent program for ``--use-agentic-rollout``: two model turns with a "tool" reply in between.

It is started once per sample with the session environment (see relax_b200/rollout/agent_runner.py): reads its input
file, talks to the policy through the chat endpoint under its session id, and writes a reward before it exits.  Any
program in any language that does the same three things can take its place."""
import json
import os
import urllib.request


def chat(messages, max_tokens):
    req = urllib.request.Request(
        os.environ["RELAX_BASE_URL"] + "/v1/chat/completions",
        data=json.dumps({"messages": messages, "max_tokens": max_tokens}).encode(),
        headers={"Content-Type": "application/json", "X-Session-Id": os.environ["RELAX_SESSION_ID"]})
    with urllib.request.urlopen(req, timeout=600) as r:
        return json.loads(r.read())["choices"][0]["message"]["content"]


def main():
    task = json.load(open(os.environ["RELAX_INPUT_JSON"]))
    budget = int(task.get("max_new_tokens") or 16)
    messages = [{"role": "user", "content": str(task["prompt"])}]
    first = chat(messages, budget)
    messages += [{"role": "assistant", "content": first}, {"role": "user", "content": f"tool: your reply had {len(first)} characters"}]
    second = chat(messages, budget)
    # a toy reward: shorter final answers score higher
    json.dump({"reward": 1.0 / (1.0 + len(second)), "metadata": {"first_len": len(first), "second_len": len(second)}},
              open(os.environ["RELAX_OUTPUT_JSON"], "w"))


if __name__ == "__main__":
    main()
