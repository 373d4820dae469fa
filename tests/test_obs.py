"""Observability: loop timers, request stamps, the native-load log, and their appearance on /health."""

import time

import requests
from http_util import ServerProc


def test_loop_timers_file_stages_by_kind_and_batch(monkeypatch):
    from b200serve.obs import looptimers as lt

    monkeypatch.setattr(lt, "ENABLED", True)
    lt.reset()
    for batch, with_prefill in ((4, False), (4, False), (4, True), (16, False)):
        lt.begin()
        if with_prefill:
            with lt.stage("prefill"):
                time.sleep(0.002)
        with lt.stage("decode"):
            time.sleep(0.001)
        lt.add("build", 0.0005)
        lt.add("build", 0.0005)  # the same stage twice in one iteration adds up
        lt.end(batch)
    lt.begin()
    lt.end(4)  # an iteration that did nothing is not recorded
    s = lt.summary()
    assert set(s) == {"pure:b4", "mixed:b4", "pure:b16"}
    assert s["pure:b4"]["decode"]["n"] == 2 and s["mixed:b4"]["prefill"]["n"] == 1
    assert 0.9 <= s["pure:b4"]["build"]["p50_ms"] <= 1.1
    assert s["mixed:b4"]["total"]["mean_ms"] >= s["mixed:b4"]["prefill"]["mean_ms"] >= 2.0
    start, stop = lt.gpu_span("gpu")  # without a device the span is a pair of no-ops
    start()
    stop()
    lt.reset()
    assert lt.summary() == {}
    monkeypatch.setattr(lt, "ENABLED", False)
    lt.begin()
    with lt.stage("decode"):
        pass
    lt.end(1)
    assert lt.summary() == {}


def test_request_stamps_report_offsets_and_the_router_hop(monkeypatch):
    from b200serve.obs import reqstamps as rs

    assert rs.start("123.0") is None or rs.ENABLED
    monkeypatch.setattr(rs, "ENABLED", True)
    rs.reset()
    st = rs.start(repr(time.time() - 0.05))
    rs.mark(st, "parsed")
    time.sleep(0.003)
    rs.mark(st, "first_byte")
    rs.finish(st)
    bad = rs.start("not a number")  # an unreadable header is ignored
    rs.finish(bad)
    rs.mark(None, "parsed")
    rs.finish(None)
    s = rs.summary()
    assert 40 <= s["router_hop"]["p50_ms"] <= 500 and s["router_hop"]["n"] == 1
    assert s["first_byte"]["p50_ms"] >= s["parsed"]["p50_ms"] and s["done"]["n"] == 2
    rs.reset()
    assert rs.summary() == {}


def test_native_load_log_separates_loads_while_serving(monkeypatch):
    from b200serve.obs import buildlog as bl

    monkeypatch.setattr(bl, "_events", [])
    monkeypatch.setattr(bl, "_serving", False)
    bl.record("load", "libkernels.so", 0.01)
    bl.mark_serving()
    bl.record("load", "late.so", 0.02)
    assert [e["what"] for e in bl.events()] == ["libkernels.so", "late.so"]
    assert [e["what"] for e in bl.events(serving_only=True)] == ["late.so"]


def test_health_carries_timers_and_stamps_when_switched_on():
    s = ServerProc("random:tiny", env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_LOOP_TIMERS": "1", "ENGINE_REQ_STAMPS": "1"})
    try:
        body = {"model": s.model, "prompt": list(range(10, 50)), "max_tokens": 6, "temperature": 0, "ignore_eos": True}
        assert s.post("/v1/completions", body).status_code == 200
        s.completion(list(range(10, 60)), 5)
        h = requests.get(s.url + "/health", timeout=10).json()
        timers, stamps = h["loop_timers"], h["request_stamps"]
        assert any(k.startswith(("pure:", "mixed:")) for k in timers)
        assert any("decode" in v or "prefill" in v for v in timers.values())
        assert {"parsed", "tokenized", "first_event", "done"} <= set(stamps) and stamps["done"]["n"] == 2
        assert stamps["first_byte"]["n"] == 1  # only the streamed request has a first byte of its own
        assert h["native_loads_while_serving"] == 0
    finally:
        s.stop()


def test_metrics_endpoint_mirrors_the_numeric_health_fields():
    from b200serve.api.server import metrics_text

    text = metrics_text({"status": "ok", "decode_steps": 12, "kv_pages_free": 7.5, "broken": None, "flag": True, "odd key-name": 3})
    assert "engine_up 1\n" in text and "engine_decode_steps 12\n" in text and "engine_kv_pages_free 7.5\n" in text
    assert "engine_odd_key_name 3\n" in text and "flag" not in text and "broken" not in text
    assert "engine_up 0\n" in metrics_text({"status": "unavailable"})
    s = ServerProc("random:tiny", env={"CUDA_VISIBLE_DEVICES": ""})
    try:
        s.completion(list(range(10, 40)), 4)
        r = requests.get(s.url + "/metrics", timeout=10)
        assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
        values = dict(ln.split(" ") for ln in r.text.splitlines() if ln and not ln.startswith("#"))
        assert values["engine_up"] == "1" and int(values["engine_finished"]) == 1 and int(values["engine_decoded_tokens"]) >= 3
    finally:
        s.stop()
