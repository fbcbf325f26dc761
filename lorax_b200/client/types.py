"""Request / response types of the Python client (pydantic), mirroring the REST surface
(`clients/python/lorax/types.py` in the reference)."""

from __future__ import annotations

from enum import Enum
from typing import Any, Dict, List, Optional, Union

from pydantic import AliasChoices, BaseModel, ConfigDict, Field, field_validator, model_validator

ADAPTER_SOURCES = ["hub", "local", "s3", "pbase"]
MERGE_STRATEGIES = ["linear", "ties", "dare_linear", "dare_ties"]
MAJORITY_SIGN_METHODS = ["total", "frequency"]


class ValidationError(ValueError):
    pass


class MergedAdapters(BaseModel):
    ids: List[str]
    weights: List[float]
    merge_strategy: Optional[str] = None
    density: float = 0.0
    majority_sign_method: Optional[str] = None

    @model_validator(mode="after")
    def _check(self):
        if len(self.ids) != len(self.weights):
            raise ValidationError("`ids` and `weights` must have the same length")
        if len(self.ids) < 1:
            raise ValidationError("`ids` cannot be empty")
        if self.merge_strategy is not None and self.merge_strategy not in MERGE_STRATEGIES:
            raise ValidationError(f"`merge_strategy` must be one of {MERGE_STRATEGIES}")
        if not 0.0 <= self.density <= 1.0:
            raise ValidationError("`density` must be >= 0.0 and <= 1.0")
        if self.majority_sign_method is not None and self.majority_sign_method not in MAJORITY_SIGN_METHODS:
            raise ValidationError(f"`majority_sign_method` must be one of {MAJORITY_SIGN_METHODS}")
        return self


class ResponseFormatType(str, Enum):
    json_object = "json_object"
    json_schema = "json_schema"
    text = "text"


class ResponseFormat(BaseModel):
    # `ResponseFormat(type="json_object", schema={...})`, as with the reference client (types.py:65-71 there names the field
    # `schema_spec` with the same alias); `schema_=` and `schema_spec=` are accepted too
    model_config = ConfigDict(populate_by_name=True)

    type: ResponseFormatType
    schema_: Optional[Union[Dict[str, Any], str]] = Field(None, validation_alias=AliasChoices("schema", "schema_", "schema_spec"))

    @property
    def schema_spec(self):
        return self.schema_

    def to_dict(self):
        d: Dict[str, Any] = {"type": self.type.value}
        if self.schema_ is not None:
            d["schema"] = self.schema_
        return d


class Parameters(BaseModel):
    adapter_id: Optional[str] = None
    adapter_source: Optional[str] = None
    merged_adapters: Optional[MergedAdapters] = None
    api_token: Optional[str] = None
    do_sample: bool = False
    max_new_tokens: Optional[int] = None
    ignore_eos_token: bool = False
    repetition_penalty: Optional[float] = None
    frequency_penalty: Optional[float] = None
    presence_penalty: Optional[float] = None
    return_full_text: bool = False
    stop: List[str] = []
    seed: Optional[int] = None
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    truncate: Optional[int] = None
    typical_p: Optional[float] = None
    best_of: Optional[int] = None
    watermark: bool = False
    details: bool = False
    decoder_input_details: bool = False
    return_k_alternatives: Optional[int] = None
    response_format: Optional[Dict[str, Any]] = None

    @field_validator("response_format", mode="before")
    def _response_format_as_dict(cls, v):
        if isinstance(v, ResponseFormat):
            return v.to_dict()
        if isinstance(v, dict) and "type" in v:          # same checks and spelling whichever way it was given
            return ResponseFormat(**v).to_dict()
        return v

    @model_validator(mode="after")
    def _check(self):
        if self.adapter_id is not None and self.merged_adapters is not None:
            raise ValidationError("you must specify at most one of `adapter_id` or `merged_adapters`")
        if self.adapter_source is not None and self.adapter_source not in ADAPTER_SOURCES:
            raise ValidationError(f"`adapter_source` must be one of {ADAPTER_SOURCES}")
        if self.best_of is not None:
            if self.best_of <= 0:
                raise ValidationError("`best_of` must be strictly positive")
            if self.best_of > 1 and self.seed is not None:
                raise ValidationError("`seed` must not be set when `best_of` is > 1")
            sampling = self.do_sample or self.temperature is not None or self.top_k is not None or self.top_p is not None or self.typical_p is not None
            if self.best_of > 1 and not sampling:
                raise ValidationError("you must use sampling when `best_of` is > 1")
        if self.repetition_penalty is not None and self.repetition_penalty <= 0:
            raise ValidationError("`repetition_penalty` must be strictly positive")
        for name in ("frequency_penalty", "presence_penalty"):
            v = getattr(self, name)
            if v is not None and not -2.0 <= v <= 2.0:
                raise ValidationError(f"`{name}` must be >= -2.0 and <= 2.0")
        if self.seed is not None and self.seed < 0:
            raise ValidationError("`seed` must be positive")
        if self.temperature is not None and self.temperature < 0:
            raise ValidationError("`temperature` must be non-negative")
        if self.top_k is not None and self.top_k <= 0:
            raise ValidationError("`top_k` must be strictly positive")
        if self.top_p is not None and not 0 < self.top_p <= 1:
            raise ValidationError("`top_p` must be > 0.0 and <= 1.0")
        if self.truncate is not None and self.truncate <= 0:
            raise ValidationError("`truncate` must be strictly positive")
        if self.typical_p is not None and not 0 < self.typical_p < 1:
            raise ValidationError("`typical_p` must be > 0.0 and < 1.0")
        if self.return_k_alternatives is not None and self.return_k_alternatives <= 0:
            raise ValidationError("`return_k_alternatives` must be strictly positive")
        return self


class Request(BaseModel):
    inputs: str
    parameters: Optional[Parameters] = None
    stream: bool = False

    @model_validator(mode="after")
    def _check(self):
        if not self.inputs:
            raise ValidationError("`inputs` cannot be empty")
        if self.stream and self.parameters is not None and self.parameters.best_of is not None and self.parameters.best_of > 1:
            raise ValidationError("`best_of` != 1 is not supported when `stream` == True")
        return self


class BatchRequest(BaseModel):
    """Several prompts under one set of parameters (`clients/python/lorax/types.py:238-250` of the reference)."""
    inputs: List[str]
    parameters: Optional[Parameters] = None
    stream: bool = False

    @field_validator("inputs")
    def _not_empty(cls, v):
        if not v:
            raise ValidationError("`inputs` cannot be empty")
        return v


class DeployedModel(BaseModel):
    model_config = ConfigDict(protected_namespaces=())
    model_id: str
    sha: str


class InputToken(BaseModel):
    id: int
    text: str
    logprob: Optional[float] = None


class AlternativeToken(BaseModel):
    id: int
    text: str
    logprob: float


class Token(BaseModel):
    id: int
    text: str
    logprob: Optional[float] = None
    special: bool = False
    alternative_tokens: Optional[List[AlternativeToken]] = None
    skipped: bool = False


class FinishReason(str, Enum):
    Length = "length"
    EndOfSequenceToken = "eos_token"
    StopSequence = "stop_sequence"


class BestOfSequence(BaseModel):
    generated_text: str
    finish_reason: FinishReason
    generated_tokens: int
    seed: Optional[int] = None
    prefill: List[InputToken] = []
    tokens: List[Token] = []


class Details(BaseModel):
    finish_reason: FinishReason
    prompt_tokens: int = 0
    generated_tokens: int
    skipped_tokens: int = 0
    seed: Optional[int] = None
    prefill: List[InputToken] = []
    tokens: List[Token] = []
    best_of_sequences: Optional[List[BestOfSequence]] = None


class Response(BaseModel):
    generated_text: str
    details: Optional[Details] = None


class StreamDetails(BaseModel):
    finish_reason: FinishReason
    generated_tokens: int
    skipped_tokens: int = 0
    seed: Optional[int] = None


class StreamResponse(BaseModel):
    token: Token
    generated_text: Optional[str] = None
    details: Optional[StreamDetails] = None


class EmbedResponse(BaseModel):
    embeddings: Optional[List[float]] = None


class ClassifyResponse(BaseModel):
    entities: Optional[List[dict]] = None
