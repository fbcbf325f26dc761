"""Synchronous and asyncio clients of the REST API: generate, generate_stream (SSE), embed, classify,
classify_batch, metrics, info, health.  Same call signatures as the reference client
(`clients/python/lorax/client.py:41-992`), so `from lorax_b200.client import Client` is a drop-in replacement."""

from __future__ import annotations

import json
from typing import Any, AsyncIterator, Dict, Iterator, List, Optional

import requests

from .errors import parse_error
from .types import (ClassifyResponse, EmbedResponse, MergedAdapters, Parameters, Request, Response, StreamResponse)

LORAX_DEBUG_MODE = False


def _parameters(**kw) -> Parameters:
    rf = kw.pop("response_format", None)
    if rf is not None and not isinstance(rf, dict):
        rf = rf.to_dict()
    ma = kw.pop("merged_adapters", None)
    if isinstance(ma, dict):
        ma = MergedAdapters(**ma)
    return Parameters(response_format=rf, merged_adapters=ma, **kw)


class Client:
    def __init__(self, base_url: str, headers: Optional[Dict[str, str]] = None, cookies: Optional[Dict[str, str]] = None,
                 timeout: int = 60, session: Optional[requests.Session] = None, max_session_retries: int = 2):
        self.base_url = base_url.rstrip("/")
        self.embed_endpoint = f"{self.base_url}/embed"
        self.classify_endpoint = f"{self.base_url}/classify"
        self.classify_batch_endpoint = f"{self.base_url}/classify_batch"
        self.headers = headers
        self.cookies = cookies
        self.timeout = timeout
        self.session = session
        self.max_session_retries = max_session_retries

    def _post(self, url: str, json_body: dict, stream: bool = False):
        s = self.session or requests
        last = None
        for _ in range(self.max_session_retries + 1):
            try:
                return s.post(url, json=json_body, headers=self.headers, cookies=self.cookies, timeout=self.timeout, stream=stream)
            except (requests.exceptions.ConnectionError, requests.exceptions.ChunkedEncodingError) as e:
                last = e
                if self.session is not None:
                    self.session.close()
                    self.session = requests.Session()
        raise last

    def generate(self, prompt: str, adapter_id: Optional[str] = None, adapter_source: Optional[str] = None,
                 merged_adapters: Optional[MergedAdapters] = None, api_token: Optional[str] = None, do_sample: bool = False,
                 max_new_tokens: Optional[int] = None, ignore_eos_token: bool = False, best_of: Optional[int] = None,
                 repetition_penalty: Optional[float] = None, frequency_penalty: Optional[float] = None,
                 presence_penalty: Optional[float] = None, return_full_text: bool = False, seed: Optional[int] = None,
                 stop_sequences: Optional[List[str]] = None, temperature: Optional[float] = None, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, truncate: Optional[int] = None, typical_p: Optional[float] = None, watermark: bool = False,
                 response_format: Optional[Any] = None, decoder_input_details: bool = False, return_k_alternatives: Optional[int] = None,
                 details: bool = True) -> Response:
        params = _parameters(adapter_id=adapter_id, adapter_source=adapter_source, merged_adapters=merged_adapters, api_token=api_token,
                             best_of=best_of, details=details, do_sample=do_sample, max_new_tokens=max_new_tokens,
                             ignore_eos_token=ignore_eos_token, repetition_penalty=repetition_penalty, frequency_penalty=frequency_penalty,
                             presence_penalty=presence_penalty, return_full_text=return_full_text, seed=seed, stop=stop_sequences or [],
                             temperature=temperature, top_k=top_k, top_p=top_p, truncate=truncate, typical_p=typical_p, watermark=watermark,
                             response_format=response_format, decoder_input_details=decoder_input_details,
                             return_k_alternatives=return_k_alternatives)
        req = Request(inputs=prompt, stream=False, parameters=params)
        resp = self._post(self.base_url + "/generate", req.model_dump(by_alias=True, exclude_none=True))
        try:
            payload = resp.json()
        except requests.JSONDecodeError as e:
            raise Exception(f"could not parse the response ({resp.status_code}): {resp.text[:200]}") from e
        if resp.status_code != 200:
            raise parse_error(resp.status_code, payload)
        return Response(**payload)

    def generate_stream(self, prompt: str, **kw) -> Iterator[StreamResponse]:
        stop = kw.pop("stop_sequences", None)
        kw.pop("best_of", None)
        params = _parameters(stop=stop or [], details=kw.pop("details", True), **kw)
        req = Request(inputs=prompt, stream=True, parameters=params)
        resp = self._post(self.base_url + "/generate_stream", req.model_dump(by_alias=True, exclude_none=True), stream=True)
        if resp.status_code != 200:
            raise parse_error(resp.status_code, resp.json())
        for byte_payload in resp.iter_lines():
            if byte_payload in (b"", b"\n"):
                continue
            payload = byte_payload.decode("utf-8")
            if payload.startswith("data:"):
                data = json.loads(payload[5:].strip())
                if "error" in data and "token" not in data:
                    raise parse_error(resp.status_code, data)
                yield StreamResponse(**data)

    def embed(self, inputs: str) -> EmbedResponse:
        resp = self._post(self.embed_endpoint, {"inputs": inputs})
        payload = resp.json()
        if resp.status_code != 200:
            raise parse_error(resp.status_code, payload)
        return EmbedResponse(**payload)

    def classify(self, inputs: str) -> ClassifyResponse:
        resp = self._post(self.classify_endpoint, {"inputs": inputs})
        payload = resp.json()
        if resp.status_code != 200:
            raise parse_error(resp.status_code, payload)
        return ClassifyResponse(entities=payload)

    def classify_batch(self, inputs: List[str]) -> List[ClassifyResponse]:
        resp = self._post(self.classify_batch_endpoint, {"inputs": inputs})
        payload = resp.json()
        if resp.status_code != 200:
            raise parse_error(resp.status_code, payload)
        return [ClassifyResponse(entities=e) for e in payload]

    def info(self) -> dict:
        return requests.get(self.base_url + "/info", headers=self.headers, timeout=self.timeout).json()

    def health(self) -> bool:
        return requests.get(self.base_url + "/health", headers=self.headers, timeout=self.timeout).status_code == 200

    def metrics(self, format: Optional[str] = None) -> str:
        url = self.base_url + "/metrics" + (f"?format={format}" if format else "")
        return requests.get(url, headers=self.headers, timeout=self.timeout).text


class AsyncClient:
    def __init__(self, base_url: str, headers: Optional[Dict[str, str]] = None, cookies: Optional[Dict[str, str]] = None, timeout: int = 60):
        from aiohttp import ClientTimeout
        self.base_url = base_url.rstrip("/")
        self.headers, self.cookies = headers, cookies
        self.timeout = ClientTimeout(timeout)

    async def generate(self, prompt: str, **kw) -> Response:
        from aiohttp import ClientSession
        stop = kw.pop("stop_sequences", None)
        params = _parameters(stop=stop or [], details=kw.pop("details", True), **kw)
        req = Request(inputs=prompt, stream=False, parameters=params)
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.post(self.base_url + "/generate", json=req.model_dump(by_alias=True, exclude_none=True)) as resp:
                payload = await resp.json()
                if resp.status != 200:
                    raise parse_error(resp.status, payload)
                return Response(**payload)

    async def generate_stream(self, prompt: str, **kw) -> AsyncIterator[StreamResponse]:
        from aiohttp import ClientSession
        stop = kw.pop("stop_sequences", None)
        kw.pop("best_of", None)
        params = _parameters(stop=stop or [], details=kw.pop("details", True), **kw)
        req = Request(inputs=prompt, stream=True, parameters=params)
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.post(self.base_url + "/generate_stream", json=req.model_dump(by_alias=True, exclude_none=True)) as resp:
                if resp.status != 200:
                    raise parse_error(resp.status, await resp.json())
                async for byte_payload in resp.content:
                    if byte_payload in (b"\n", b"\r\n", b""):
                        continue
                    payload = byte_payload.decode("utf-8").strip()
                    if payload.startswith("data:"):
                        data = json.loads(payload[5:].strip())
                        if "error" in data and "token" not in data:
                            raise parse_error(resp.status, data)
                        yield StreamResponse(**data)

    async def embed(self, inputs: str) -> EmbedResponse:
        from aiohttp import ClientSession
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.post(self.base_url + "/embed", json={"inputs": inputs}) as resp:
                payload = await resp.json()
                if resp.status != 200:
                    raise parse_error(resp.status, payload)
                return EmbedResponse(**payload)

    async def _post_json(self, path: str, body: dict):
        from aiohttp import ClientSession
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.post(self.base_url + path, json=body) as resp:
                payload = await resp.json()
                if resp.status != 200:
                    raise parse_error(resp.status, payload)
                return payload

    async def classify(self, inputs: str) -> ClassifyResponse:
        """Token classification of one text (entities when the model's labels follow the B- / I- scheme)."""
        return ClassifyResponse(entities=await self._post_json("/classify", {"inputs": inputs}))

    async def classify_batch(self, inputs: List[str]) -> List[ClassifyResponse]:
        return [ClassifyResponse(entities=e) for e in await self._post_json("/classify_batch", {"inputs": inputs})]

    async def info(self) -> dict:
        from aiohttp import ClientSession
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.get(self.base_url + "/info") as resp:
                return await resp.json()

    async def health(self) -> bool:
        from aiohttp import ClientSession
        async with ClientSession(headers=self.headers, cookies=self.cookies, timeout=self.timeout) as session:
            async with session.get(self.base_url + "/health") as resp:
                return resp.status == 200
