from .client import AsyncClient, Client  # noqa: F401
from .types import BatchRequest, DeployedModel, MergedAdapters, Parameters, Request, Response, ResponseFormat, StreamResponse  # noqa: F401
