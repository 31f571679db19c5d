"""Rollout dumps and the viewer (CPU; the HTTP server runs on a loopback port chosen by the OS)."""
import json
import urllib.request

from relax_b200.types import Sample, SampleStatus
from relax_b200.utils import visualize as V


def _samples():
    out = []
    for g in range(2):
        for k in range(3):
            out.append(Sample(group_index=g, index=g * 3 + k, prompt=f"q{g} <b>", tokens=[1, 2, 3, 4 + k, 5], response=f"ans {k} & more",
                              response_length=2, reward=float(k == 1) if g == 0 else 1.0, rollout_log_probs=[-0.1, -4.0],
                              loss_mask=[1, 0], status=SampleStatus.TRUNCATED if k == 2 else SampleStatus.COMPLETED))
    return out


def test_dump_summary_text_and_html(tmp_path):
    d = str(tmp_path)
    V.dump_rollout(d, 0, _samples(), extra={"weight_version": 3})
    V.dump_rollout(d, 1, [s.to_dict() for s in _samples()[:3]])
    assert V.list_steps(d) == [0, 1]
    header, samples = V.load_step(d, 0)
    assert header["weight_version"] == 3 and len(samples) == 6 and samples[0]["status"] == "completed"
    sm = V.step_summary(samples)
    assert sm["samples"] == 6 and sm["truncated"] == 2 and sm["groups"] == 2 and sm["zero_std_groups"] == 1
    assert abs(sm["reward_mean"] - 4 / 6) < 1e-9
    txt = V.render_text(d)
    assert txt.splitlines()[1].split()[0] == "0" and "1/2" in txt
    assert "ans 1" in V.render_text(d, 0)
    page = V.render_sample(d, 0, 1, decode_token=lambda t: f"<{t}>")
    assert "&lt;5&gt;" in page and "q0 &lt;b&gt;" in page and "opacity" in page     # escaped, masked token faded
    assert "sort=reward" in V.render_step(d, 0, "reward")


def test_http_routes(tmp_path):
    d = str(tmp_path)
    V.dump_rollout(d, 7, _samples())
    srv, th = V.serve_in_thread(d)
    try:
        base = f"http://127.0.0.1:{srv.server_address[1]}"
        assert "/step?id=7" in urllib.request.urlopen(base + "/").read().decode()
        assert "ans 2 &amp; more" in urllib.request.urlopen(base + "/step?id=7&sort=length").read().decode()
        assert "rollout log-prob" in urllib.request.urlopen(base + "/sample?id=7&n=0").read().decode()
        api = json.loads(urllib.request.urlopen(base + "/api/steps").read())
        assert api["7"]["samples"] == 6
        try:
            urllib.request.urlopen(base + "/step?id=99")
            assert False
        except urllib.error.HTTPError as e:
            assert e.code == 400
    finally:
        srv.shutdown()
        srv.server_close()


def test_decode_fills_missing_text(tmp_path):
    s = Sample(tokens=[10, 11, 12, 13], response_length=2, prompt=[10, 11])
    V.dump_rollout(str(tmp_path), 0, [s], decode=lambda ids: " ".join(map(str, ids)))
    _, (row,) = V.load_step(str(tmp_path), 0)
    assert row["response"] == "12 13" and row["prompt"] == "10 11"
    assert V.main(["--dir", str(tmp_path), "--text"]) == 0
