"""HTTP error payloads -> exceptions (same mapping as `clients/python/lorax/errors.py` of the reference)."""

from typing import Dict


class ValidationError(Exception):
    pass


class GenerationError(Exception):
    pass


class OverloadedError(Exception):
    pass


class IncompleteGenerationError(Exception):
    pass


class BadRequestError(Exception):
    pass


class ShardNotReadyError(Exception):
    pass


class ShardTimeoutError(Exception):
    pass


class NotFoundError(Exception):
    pass


class RateLimitExceededError(Exception):
    pass


class NotSupportedError(Exception):
    def __init__(self, model_id: str):
        super().__init__(f"Model `{model_id}` is not available for inference with this client.")


class UnknownError(Exception):
    pass


def parse_error(status_code: int, payload: Dict[str, str]) -> Exception:
    message = payload.get("error", "")
    error_type = payload.get("error_type")
    if error_type == "generation":
        return GenerationError(message)
    if error_type == "incomplete_generation":
        return IncompleteGenerationError(message)
    if error_type == "overloaded":
        return OverloadedError(message)
    if error_type == "validation":
        return ValidationError(message)
    if status_code == 400:
        return BadRequestError(message)
    if status_code in (403, 424):
        return ShardNotReadyError(message)
    if status_code == 504:
        return ShardTimeoutError(message)
    if status_code == 404:
        return NotFoundError(message)
    if status_code == 429:
        return RateLimitExceededError(message)
    return UnknownError(message)
