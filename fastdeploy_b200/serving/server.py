"""HTTP front end compatible with the reference's ``SimpleServer``
(python/fastdeploy/serving/server.py:20-60, router/http_router.py:30-85, model_manager.py:24-60,
handler/*.py): ``app.register(task_name, model_handler, predictor)`` exposes ``POST /{task_name}`` taking
``{"data": ..., "parameters": {...}}`` and answering ``{"result": ...}``; a handler is a class with a
``process(predictor, data, parameters)`` classmethod.

On top of that, ``register`` accepts a list of predictors (one per GPU) or a :class:`Scheduler`, in which
case requests are load-balanced and batched instead of serialised on one lock, and
:meth:`SimpleServer.register_repository` serves every model of a Triton-style repository through
``POST /v2/models/{name}/infer`` (KServe v2 JSON tensors).
"""
import base64
import contextlib
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .scheduler import Scheduler


@contextlib.contextmanager
def lock_predictor(lock):
    lock.acquire()
    try:
        yield
    finally:
        lock.release()


def cv2_to_base64(image: np.ndarray) -> str:
    import cv2
    return base64.b64encode(cv2.imencode(".jpg", image)[1].tobytes()).decode("utf8")


def base64_to_cv2(b64str: str) -> np.ndarray:
    import cv2
    return cv2.imdecode(np.frombuffer(base64.b64decode(b64str.encode("utf8")), np.uint8), cv2.IMREAD_COLOR)


class BaseModelHandler:
    @classmethod
    def process(cls, predictor, data, parameters):
        raise NotImplementedError


class VisionModelHandler(BaseModelHandler):
    @classmethod
    def process(cls, predictor, data, parameters):
        from ..vision.utils import fd_result_to_json
        return fd_result_to_json(predictor.predict(base64_to_cv2(data["image"])))


class ModelManager:
    def __init__(self, model_handler, predictor):
        if not (isinstance(model_handler, type) and issubclass(model_handler, BaseModelHandler)):
            raise TypeError("The model_handler must be subclass of BaseModelHandler, please check the type.")
        self._handler = model_handler
        self._scheduler: Optional[Scheduler] = predictor if isinstance(predictor, Scheduler) else None
        preds = [] if self._scheduler else (list(predictor) if isinstance(predictor, (list, tuple)) else [predictor])
        self._predictors = preds
        self._locks = [threading.Lock() for _ in preds]
        self._rr = 0

    def predict(self, data, parameters):
        if self._scheduler is not None:
            return self._scheduler.infer((data, parameters))
        self._rr = (self._rr + 1) % len(self._predictors)
        i = self._rr
        with lock_predictor(self._locks[i]):
            return self._handler.process(self._predictors[i], data, parameters)


def batched_runtime_fn(rt, payloads):
    """Execute step of the serving back end: the requests a worker took from its queue are gathered along the
    batch dimension into ONE ``Runtime.infer`` call and the outputs are sliced back per request - what the
    reference's Triton back end does with ``BackendInputCollector`` / ``BackendOutputResponder``
    (serving/src/fastdeploy_runtime.cc:1158-1313). Requests whose non-batch dimensions differ run one by one."""
    if len(payloads) == 1:
        return [rt.infer(payloads[0])]
    names = list(payloads[0].keys())
    arrays = [[np.asarray(p[n]) for n in names] for p in payloads]
    same = all(set(p.keys()) == set(names) for p in payloads) and all(
        a[k].ndim >= 1 and a[k].shape[1:] == arrays[0][k].shape[1:] and a[k].dtype == arrays[0][k].dtype
        for a in arrays for k in range(len(names)))
    rows = [a[0].shape[0] if a and a[0].ndim else 1 for a in arrays]
    same = same and all(x.shape[0] == r for a, r in zip(arrays, rows) for x in a)
    if not same:
        return [rt.infer(p) for p in payloads]
    feeds = {n: np.concatenate([a[k] for a in arrays], 0) for k, n in enumerate(names)}
    outs = rt.infer(feeds)
    total = sum(rows)
    res, pos = [], 0
    for r in rows:
        res.append([np.asarray(o)[pos:pos + r] if np.asarray(o).ndim and np.asarray(o).shape[0] == total else o
                    for o in outs])
        pos += r
    return res


_TRITON_DTYPES = {"FP32": np.float32, "FP16": np.float16, "INT64": np.int64, "INT32": np.int32, "UINT8": np.uint8,
                  "INT8": np.int8, "BOOL": np.bool_, "FP64": np.float64}


def _metric_name(name: str) -> str:
    return "".join(ch if ch.isalnum() else "_" for ch in name)


def _build_app():
    from fastapi import FastAPI, HTTPException, Request

    class SimpleServer(FastAPI):
        def __init__(self, **kwargs):
            super().__init__(**kwargs)
            self._managers: Dict[str, ModelManager] = {}
            self._runtimes: Dict[str, Any] = {}
            self._service_name = "FastDeploy SimpleServer"

            @self.get("/health")
            def health():
                return {"status": "ok", "models": sorted(list(self._managers) + list(self._runtimes))}

            @self.get("/metrics")
            def metrics():
                """Prometheus text: per model and worker request / failure / deadline counters, queue depth,
                queueing and compute time, and the histogram of executed batch sizes."""
                from fastapi.responses import PlainTextResponse
                parts = []
                for name, m in sorted(self._managers.items()):
                    if m._scheduler is not None:
                        parts.append(m._scheduler.metrics_text(prefix="fdb_" + _metric_name(name)))
                for name, (_, sched, _) in sorted(self._runtimes.items()):
                    parts.append(sched.metrics_text(prefix="fdb_" + _metric_name(name)))
                return PlainTextResponse("".join(parts), media_type="text/plain; version=0.0.4")

        def register(self, task_name: str, model_handler, predictor):
            manager = ModelManager(model_handler, predictor)
            self._managers[task_name] = manager

            async def predict(request: Request):
                body = await request.json()
                if not isinstance(body, dict) or "data" not in body or set(body) - {"data", "parameters"}:
                    raise HTTPException(status_code=422, detail="body must be {data, parameters?}")
                try:
                    result = manager.predict(body["data"], body.get("parameters") or {})
                except Exception as e:
                    raise HTTPException(status_code=400, detail=f"Error occurred while running predict: {e}")
                return {"result": result}
            self.add_api_route(f"/{task_name}", predict, methods=["POST"], summary=task_name.title())

        def register_repository(self, repo: str, device_ids: Optional[Sequence[int]] = None):
            """Loads every model of a Triton-style repository; one runtime per listed instance."""
            from ..runtime.runtime import Runtime
            from .model_repository import scan_repository
            for name, cfg in scan_repository(repo).items():
                insts = cfg.instances()
                if device_ids is not None:
                    insts = [("gpu", d) for d in device_ids]
                rts = [Runtime(cfg.runtime_option(kind, dev)) for kind, dev in insts]

                sched = Scheduler(lambda i, rts=rts: rts[i], batched_runtime_fn, num_workers=len(rts),
                                  max_batch_size=max(cfg.max_batch_size, 1), max_queue_delay_us=cfg.max_queue_delay_us)
                self._runtimes[name] = (cfg, sched, rts)
            if not getattr(self, "_v2_routes", False):
                self._v2_routes = True

                @self.get("/v2/models/{name}")
                def metadata(name: str):
                    if name not in self._runtimes:
                        raise HTTPException(status_code=404, detail="unknown model")
                    cfg = self._runtimes[name][0]
                    return {"name": cfg.name, "versions": [str(v) for v in cfg.versions()], "platform": cfg.backend,
                            "inputs": cfg.inputs, "outputs": cfg.outputs}

                @self.get("/v2/models/{name}/stats")
                def stats(name: str):
                    if name not in self._runtimes:
                        raise HTTPException(status_code=404, detail="unknown model")
                    return {"model_name": name, **self._runtimes[name][1].stats()}

                @self.post("/v2/models/{name}/infer")
                async def infer(name: str, request: Request):
                    if name not in self._runtimes:
                        raise HTTPException(status_code=404, detail="unknown model")
                    cfg, sched, rts = self._runtimes[name]
                    body = await request.json()
                    feeds = {}
                    try:
                        for t in body["inputs"]:
                            dt = _TRITON_DTYPES[t["datatype"]]
                            feeds[t["name"]] = np.asarray(t["data"], dtype=dt).reshape(t["shape"])
                        outs = sched.infer(feeds)
                    except Exception as e:
                        raise HTTPException(status_code=400, detail=str(e))
                    names = [o.name for o in rts[0].get_output_infos()]
                    inv = {v: k for k, v in _TRITON_DTYPES.items()}
                    return {"model_name": name, "outputs": [
                        {"name": n, "shape": list(np.asarray(o).shape), "datatype": inv.get(np.asarray(o).dtype.type, "FP32"),
                         "data": np.asarray(o).reshape(-1).tolist()} for n, o in zip(names, outs)]}

    return SimpleServer


def __getattr__(name):
    if name == "SimpleServer":
        cls = _build_app()
        globals()["SimpleServer"] = cls
        return cls
    raise AttributeError(name)
