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


def _body_models(task_name: str):
    """Request and response schema of one task: ``data`` and ``result`` may hold anything; schema names must be unique
    per application, so they carry a digest of the task name."""
    tag = hashlib.md5(task_name.encode()).hexdigest()
    request = create_model(f"RequestModel{tag}", __base__=RequestBase, data=(typing.Any, ...))
    response = create_model(f"ResponseModel{tag}", __base__=ResponseBase, result=(typing.Any, ...))
    return request, response


class HttpRouterManager(BaseRouterManager):
    """``app`` needs a ``_model_manager`` with ``predict(data, parameters)`` by the time a request arrives."""

    def register_models_router(self, task_name: str):
        body_cls, answer_cls = _body_models(task_name)
        owner = self._app

        # (the annotation must be the class itself: the framework reads it to find the request body)
        def serve(request: Request, payload: body_cls):     # type: ignore[valid-type]
            try:
                return {"result": owner._model_manager.predict(payload.data, payload.parameters)}
            except Exception as exc:
                raise HTTPException(status_code=400, detail=f"Error occurred while running predict: {exc}")

        routes = APIRouter()
        routes.post(f"/{task_name}", summary=task_name.title(), response_model=answer_cls, response_model_exclude_unset=True,
                    response_model_exclude_none=True)(serve)
        owner.include_router(routes)
        return routes
