"""Where model and adapter files come from: a local directory, the HuggingFace hub cache, S3, or Predibase.

Counterpart of `server/lorax_server/utils/sources/{__init__,hub,local,s3}.py`.  Every source resolves to a local
directory that holds `config.json` + `*.safetensors` (model) or `adapter_config.json` + `adapter_model.safetensors`
(adapter).  Remote sources are only reachable when the machine has network access and the client library.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Optional

HUB, S3, LOCAL, PBASE = "hub", "s3", "local", "pbase"


class SourceError(RuntimeError):
    pass


def _cache_root() -> Path:
    return Path(os.environ.get("HUGGINGFACE_HUB_CACHE") or os.environ.get("HF_HUB_CACHE") or Path.home() / ".cache/huggingface/hub")


def _hub_snapshot(repo_id: str, revision: Optional[str], api_token: Optional[str], patterns) -> str:
    # offline first: a snapshot that is already in the cache
    folder = _cache_root() / ("models--" + repo_id.replace("/", "--")) / "snapshots"
    if folder.is_dir():
        snaps = sorted(folder.iterdir(), key=lambda p: p.stat().st_mtime, reverse=True)
        for s in snaps:
            if revision is None or s.name.startswith(revision):
                return str(s)
    if os.environ.get("HF_HUB_OFFLINE") == "1":
        raise SourceError(f"{repo_id} is not in the local hub cache and HF_HUB_OFFLINE=1")
    try:
        from huggingface_hub import snapshot_download
        return snapshot_download(repo_id, revision=revision, token=api_token or os.environ.get("HUGGING_FACE_HUB_TOKEN"),
                                 allow_patterns=patterns)
    except Exception as e:  # no network, bad id, gated repo ...
        raise SourceError(f"cannot fetch {repo_id} from the hub: {e}") from e


def _s3_sync(uri: str) -> str:
    try:
        import boto3
    except ImportError as e:
        raise SourceError("the s3 source needs boto3, which is not installed") from e
    bucket_name = os.environ.get("PREDIBASE_MODEL_BUCKET", "")
    key = uri
    if uri.startswith("s3://"):
        bucket_name, _, key = uri[5:].partition("/")
    bucket = boto3.resource("s3").Bucket(bucket_name)
    dest = _cache_root() / ("models--" + key.strip("/").replace("/", "--")) / "snapshots" / "s3"
    dest.mkdir(parents=True, exist_ok=True)
    for obj in bucket.objects.filter(Prefix=key):
        rel = obj.key[len(key):].lstrip("/")
        if rel:
            target = dest / rel
            target.parent.mkdir(parents=True, exist_ok=True)
            if not target.exists():
                bucket.download_file(obj.key, str(target))
    return str(dest)


def resolve_model(model_id: str, source: str = HUB, revision: Optional[str] = None) -> str:
    if os.path.isdir(model_id):
        return model_id
    # WEIGHTS_CACHE_OVERRIDE (the launcher's --weights-cache-override): a directory that already holds the files of the model,
    # read instead of any download (utils/weights.py:460-552 of the reference checks the same variable first)
    override = os.environ.get("WEIGHTS_CACHE_OVERRIDE")
    if override and os.path.isdir(override) and os.path.exists(os.path.join(override, "config.json")):
        return override
    if source == LOCAL:
        raise SourceError(f"local model directory {model_id} does not exist")
    if source == S3:
        return _s3_sync(model_id)
    return _hub_snapshot(model_id, revision, None, ["*.json", "*.safetensors", "*.model", "*.txt", "*.bin"])


def resolve_adapter(adapter_id: str, source: str = HUB, api_token: Optional[str] = None, revision: Optional[str] = None) -> str:
    if os.path.isdir(adapter_id):
        medusa = any(os.path.exists(os.path.join(adapter_id, f)) for f in ("medusa_lm_head.safetensors", "medusa_lm_head.pt"))
        if not os.path.exists(os.path.join(adapter_id, "adapter_config.json")) and not medusa:
            raise SourceError(f"{adapter_id} has neither adapter_config.json (LoRA) nor medusa_lm_head.* (Medusa)")
        return adapter_id
    if source == LOCAL:
        raise SourceError(f"local adapter directory {adapter_id} does not exist")
    if source == S3:
        return _s3_sync(adapter_id)
    if source == PBASE:
        gateway = os.environ.get("PREDIBASE_GATEWAY_ENDPOINT")
        api_token = api_token or os.environ.get("PREDIBASE_API_TOKEN")      # the launcher's --predibase-api-token
        if not gateway:
            raise SourceError("the pbase source needs PREDIBASE_GATEWAY_ENDPOINT and an api_token")
        import requests
        name, _, version = adapter_id.partition("/")
        r = requests.get(f"{gateway}/v2/repos/{name}/version/{version or 'latest'}", headers={"Authorization": f"Bearer {api_token}"}, timeout=30)
        r.raise_for_status()
        return _s3_sync(r.json()["adapterPath"])
    return _hub_snapshot(adapter_id, revision, api_token, ["adapter_config.json", "adapter_model.*", "tokenizer*", "config.json", "medusa_lm_head.*"])
