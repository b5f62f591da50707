"""Route registration as separate objects (python/fastdeploy/serving/router/base_router.py:19-30,
python/fastdeploy/serving/router/http_router.py:26-80): a router manager holds the application and adds one POST route per
task; the route reads ``{"data": ..., "parameters": {...}}``, calls the application's model manager and answers
``{"result": ...}``. ``SimpleServer.register`` does the same in one call; these classes are for code that builds its
own ``FastAPI`` application around a model manager."""
import abc
import hashlib
import typing
from typing import Optional

from fastapi import APIRouter, HTTPException, Request
from pydantic import BaseModel, ConfigDict, create_model


class BaseRouterManager(abc.ABC):
    _app = None

    def __init__(self, app):
        super().__init__()
        self._app = app

    @abc.abstractmethod
    def register_models_router(self, task_name: str):
        raise NotImplementedError


class ResponseBase(BaseModel):
    text: Optional[str] = None


class RequestBase(BaseModel):
    model_config = ConfigDict(extra="forbid")
    parameters: Optional[dict] = {}


class HttpRouterManager(BaseRouterManager):
    """``app`` needs a ``_model_manager`` with ``predict(data, parameters)`` by the time a request arrives."""

    def register_models_router(self, task_name: str):
        unique = hashlib.md5(task_name.encode()).hexdigest()
        req_model = create_model("RequestModel" + unique, data=(typing.Any, ...), __base__=RequestBase)
        resp_model = create_model("ResponseModel" + unique, result=(typing.Any, ...), __base__=ResponseBase)
        app = self._app

        # (annotations must be the classes themselves here: the framework reads them to find the request body)
        def predict(request: Request, inference_request: req_model):     # type: ignore[valid-type]
            try:
                result = app._model_manager.predict(inference_request.data, inference_request.parameters)
            except Exception as e:
                raise HTTPException(status_code=400, detail=f"Error occurred while running predict: {e}")
            return {"result": result}

        router = APIRouter()
        router.add_api_route(f"/{task_name}", predict, methods=["post"], summary=task_name.title(), response_model=resp_model,
                             response_model_exclude_unset=True, response_model_exclude_none=True)
        app.include_router(router)
        return router
