"""Scheduler / batcher with fake devices, config.pbtxt parsing, SimpleServer routes (in-process client)."""
import os
import threading
import time

import numpy as np
import pytest

from fastdeploy_b200.serving import Scheduler, parse_pbtxt, load_model_config


class FakeModel:
    def __init__(self, index, fail_after=None, delay=0.002):
        self.index, self.calls, self.fail_after, self.delay = index, 0, fail_after, delay

    def run(self, xs):
        self.calls += 1
        if self.fail_after is not None and self.calls > self.fail_after:
            raise RuntimeError(f"device {self.index} lost")
        time.sleep(self.delay)
        return [(self.index, x * 2) for x in xs]


def test_batches_and_balances_over_workers():
    models = {}

    def factory(i):
        models[i] = FakeModel(i)
        return models[i]
    s = Scheduler(factory, lambda m, xs: m.run(xs), num_workers=4, max_batch_size=8, max_queue_delay_us=2000)
    out = s.map(list(range(200)))
    assert [v for _, v in out] == [2 * i for i in range(200)]
    st = s.stats()["workers"]
    assert all(w["requests"] > 0 for w in st) and sum(w["requests"] for w in st) == 200
    assert max(w["avg_batch_size"] for w in st) > 1.5
    s.close()


def test_failed_worker_leaves_rotation_and_requests_survive():
    def factory(i):
        if i == 3:
            raise RuntimeError("no such device")          # never joins
        return FakeModel(i, fail_after=2 if i == 1 else None)
    s = Scheduler(factory, lambda m, xs: m.run(xs), num_workers=4, max_batch_size=4, max_queue_delay_us=200, max_failures=2)
    assert len(s.alive_workers()) == 3
    ok = failed = 0
    for i in range(120):
        try:
            s.infer(i, timeout=5)
            ok += 1
        except RuntimeError:
            failed += 1
    assert failed >= 2 and ok >= 100
    assert not s.workers[1].alive and len(s.alive_workers()) == 2
    assert s.infer(7, timeout=5)[1] == 14                 # still serving
    s.close()


def test_dying_worker_hands_its_queue_over_without_a_later_submit():
    """Worker 0 dies with several requests still queued and nobody calls submit() afterwards: the queued
    requests must still complete (on worker 1), because the dying worker drains its own queue."""
    gate = threading.Event()

    class Slow(FakeModel):
        def run(self, xs):
            if self.index == 0:
                gate.wait(5)
                raise RuntimeError("device 0 lost")
            return super().run(xs)
    s = Scheduler(lambda i: Slow(i), lambda m, xs: m.run(xs), num_workers=2, max_batch_size=1,
                  max_queue_delay_us=0, max_failures=1)
    futs = [s.submit(i) for i in range(8)]           # alternate between the two workers; worker 0 is stuck
    time.sleep(0.05)
    assert s.workers[0].pending() >= 2
    gate.set()                                       # worker 0 fails its first request and dies
    done = failed = 0
    for f in futs:
        try:
            f.result(timeout=5)                      # would block for ever if the queue were left behind
            done += 1
        except RuntimeError:
            failed += 1
    assert failed == 1 and done == 7
    assert not s.workers[0].alive
    s.close()


def test_deadline_cancellation_pipelining_and_metrics():
    release = threading.Event()

    class Handle:
        def __init__(self, xs):
            self.xs = xs

        def result(self):
            return [x + 1 for x in self.xs]

    def batch_fn(m, xs):
        if xs and xs[0] == "block":
            release.wait(5)
            return ["unblocked"] * len(xs)
        return Handle(xs)                                 # asynchronous handle: resolved later, in order
    s = Scheduler(lambda i: object(), batch_fn, num_workers=1, max_batch_size=4, max_queue_delay_us=100,
                  pipeline_depth=3)
    blocker = s.submit("block")
    time.sleep(0.05)                                      # the only worker is now stuck inside batch_fn
    late = s.submit(1, timeout=0.05)                      # deadline passes while it is queued
    cancelled = s.submit(2)
    assert cancelled.cancel()                             # never started: the future can be cancelled
    time.sleep(0.1)
    release.set()
    assert blocker.result(5) == "unblocked"
    with pytest.raises(TimeoutError):
        late.result(5)
    assert s.map(list(range(20)), timeout=5) == [i + 1 for i in range(20)]
    text = s.metrics_text()
    assert 'fdb_scheduler_expired_total{worker="0"} 1' in text
    assert 'fdb_scheduler_batch_size_bucket{worker="0",le="+Inf"}' in text
    st = s.stats()["workers"][0]
    assert st["requests"] >= 21 and st["expired"] == 1 and sum(st["batch_histogram"].values()) == st["batches"]
    s.close()
    with pytest.raises(RuntimeError, match="closed"):
        s.submit(3)


def test_repository_execute_step_batches_requests():
    from fastdeploy_b200.serving.server import batched_runtime_fn

    class FakeRuntime:
        calls = []

        def infer(self, feeds):
            self.calls.append({k: v.shape for k, v in feeds.items()})
            return [feeds["x"] * 2.0, feeds["x"].sum(axis=1)]
    rt = FakeRuntime()
    reqs = [{"x": np.full((n, 3), float(n), np.float32)} for n in (1, 2, 4)]
    outs = batched_runtime_fn(rt, reqs)
    assert rt.calls == [{"x": (7, 3)}]                     # one inference for the three requests
    assert [o[0].shape for o in outs] == [(1, 3), (2, 3), (4, 3)]
    assert np.allclose(outs[2][0], 8.0) and np.allclose(outs[1][1], 6.0)
    outs = batched_runtime_fn(rt, [{"x": np.zeros((1, 3), np.float32)}, {"x": np.zeros((1, 5), np.float32)}])
    assert len(rt.calls) == 3 and outs[1][0].shape == (1, 5)   # shapes differ: run one by one


def test_all_workers_dead_is_an_error_not_a_hang():
    with pytest.raises(RuntimeError, match="no worker could be started"):
        Scheduler(lambda i: (_ for _ in ()).throw(RuntimeError("gone")), lambda m, xs: xs, num_workers=2)


PBTXT = '''
name: "ppyoloe"   # comment
backend: "fastdeploy"
max_batch_size: 16
input [
  { name: "image", data_type: TYPE_FP32, dims: [ 3, -1, -1 ] },
  { name: "scale_factor", data_type: TYPE_FP32, dims: [ 2 ] }
]
output [ { name: "multiclass_nms3_0.tmp_0", data_type: TYPE_FP32, dims: [ -1, 6 ] } ]
instance_group [ { count: 2, kind: KIND_GPU, gpus: [0, 1] } ]
dynamic_batching { preferred_batch_size: [ 4, 8 ], max_queue_delay_microseconds: 300 }
optimization { execution_accelerators { gpu_execution_accelerator : [ {
  name: "tensorrt"
  parameters { key: "precision" value: "trt_fp16" }
  parameters { key: "max_shape" value: "image:16 3 640 640" }
} ] } }
parameters { key: "note" value: { string_value: "hello" } }
'''


def test_config_pbtxt(tmp_path):
    cfg = parse_pbtxt(PBTXT)
    assert cfg["name"] == "ppyoloe" and cfg["max_batch_size"] == 16 and cfg["input"][0]["dims"] == [3, -1, -1]
    d = tmp_path / "ppyoloe"
    (d / "1").mkdir(parents=True)
    (d / "config.pbtxt").write_text(PBTXT)
    (d / "1" / "model.onnx").write_bytes(b"")
    mc = load_model_config(str(d))
    assert mc.instances() == [("gpu", 0), ("gpu", 0), ("gpu", 1), ("gpu", 1)]
    assert mc.dynamic_batching and mc.max_queue_delay_us == 300 and mc.preferred_batch_size == [4, 8]
    assert mc.parameters["note"] == "hello" and mc.versions() == [1]
    assert mc.gpu_accelerators[0]["name"] == "tensorrt"
    opt = mc.runtime_option("cpu", -1)
    assert opt.model_file.endswith("model.onnx")


def test_simple_server_routes():
    fastapi = pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient
    from fastdeploy_b200.serving import BaseModelHandler, SimpleServer

    class EchoHandler(BaseModelHandler):
        @classmethod
        def process(cls, predictor, data, parameters):
            return {"sum": predictor(data["values"]), "scale": parameters.get("scale", 1)}

    app = SimpleServer()
    app.register("add", EchoHandler, [sum, sum])
    try:
        c = TestClient(app)
    except RuntimeError as e:          # httpx is not installed in every image
        pytest.skip(str(e))
    r = c.post("/add", json={"data": {"values": [1, 2, 3]}, "parameters": {"scale": 2}})
    assert r.status_code == 200 and r.json() == {"result": {"sum": 6, "scale": 2}}
    assert c.post("/add", json={"data": {"values": ["x", 1]}}).status_code == 400
    assert c.post("/add", json={"nope": 1}).status_code == 422
    assert c.get("/health").json()["models"] == ["add"]


def test_request_future_semantics():
    """The scheduler's light future behaves like concurrent.futures.Future where callers can see it."""
    import concurrent.futures as cf
    from fastdeploy_b200.serving.scheduler import RequestFuture
    f = RequestFuture()
    assert not f.done() and not f.running() and not f.cancelled()
    with pytest.raises(TimeoutError):
        f.result(0.01)
    seen = []
    f.add_done_callback(lambda fut: seen.append(fut.result()))
    assert f.set_running_or_notify_cancel() and f.running() and not f.cancel()      # a running request stays
    threading.Timer(0.02, lambda: f.set_result(41)).start()
    assert f.result(5) == 41 and f.done() and seen == [41] and f.exception() is None
    f.set_result(99)                                                                # a second result is ignored
    assert f.result() == 41
    late = []
    f.add_done_callback(lambda fut: late.append(1))                                 # already done: called at once
    assert late == [1]
    g = RequestFuture()
    g.set_exception(ValueError("boom"))
    assert isinstance(g.exception(), ValueError)
    with pytest.raises(ValueError):
        g.result()
    h = RequestFuture()
    waiter = threading.Thread(target=lambda: seen.append("woken" if h.cancelled() or _wait_cancel(h) else "no"))
    waiter.start()
    time.sleep(0.02)
    assert h.cancel() and h.cancelled() and h.done() and not h.set_running_or_notify_cancel()
    waiter.join(5)
    assert "woken" in seen
    with pytest.raises(cf.CancelledError):
        h.result()


def _wait_cancel(fut):
    import concurrent.futures as cf
    try:
        fut.result(5)
    except cf.CancelledError:
        return True
    return False


def test_router_manager_adds_a_task_route_to_a_plain_application():
    fastapi = pytest.importorskip("fastapi")
    import fastdeploy_b200 as fd
    from fastdeploy_b200.serving import BaseRouterManager, HttpRouterManager, ModelManager, RequestBase, ResponseBase
    from fastdeploy_b200.serving.handler import BaseModelHandler as H2
    from fastdeploy_b200.serving.utils import base64_to_cv2, cv2_to_base64

    class Handler(fd.serving.BaseModelHandler):
        @classmethod
        def process(cls, predictor, data, parameters):
            return {"n": predictor(data), "p": parameters}

    assert H2 is fd.serving.BaseModelHandler and issubclass(HttpRouterManager, BaseRouterManager)
    with pytest.raises(TypeError):
        BaseRouterManager(None)                          # abstract
    app = fastapi.FastAPI()
    app._model_manager = ModelManager(Handler, len)
    HttpRouterManager(app).register_models_router("fd/count")
    assert any(getattr(r, "path", "") == "/fd/count" for r in app.routes)
    assert RequestBase(parameters={"a": 1}).parameters == {"a": 1} and ResponseBase().text is None
    with pytest.raises(Exception):
        RequestBase(parameters={}, other=1)              # unknown keys are refused
    try:
        from fastapi.testclient import TestClient
        c = TestClient(app)
    except RuntimeError as e:
        pytest.skip(str(e))
    r = c.post("/fd/count", json={"data": [1, 2, 3], "parameters": {"k": 2}})
    assert r.status_code == 200 and r.json() == {"result": {"n": 3, "p": {"k": 2}}}
    assert c.post("/fd/count", json={"data": 5}).status_code == 400           # len(5) raises inside the handler
    assert c.post("/fd/count", json={"data": [1], "extra": 1}).status_code == 422
    im = np.arange(48, dtype=np.uint8).reshape(4, 4, 3)
    assert base64_to_cv2(cv2_to_base64(im)).shape == (4, 4, 3)
