"""Python client without a server: request validation rules and the mapping of error payloads to exceptions (the reference keeps
the same two test files, clients/python/tests/test_types.py and test_errors.py)."""
import pytest

from lorax_b200.client import errors
from lorax_b200.client.types import MergedAdapters, Parameters, Request, ResponseFormat, ResponseFormatType, ValidationError


def _bad(**kw):
    with pytest.raises(Exception) as e:
        Parameters(**kw)
    assert isinstance(e.value, (ValidationError, ValueError))


def test_parameters_validation_rules():
    Parameters()                                                       # every default is valid
    Parameters(adapter_id="a/b", adapter_source="hub", do_sample=True, temperature=0.7, top_k=10, top_p=0.9, typical_p=0.5, seed=3,
               repetition_penalty=1.1, frequency_penalty=-2.0, presence_penalty=2.0, truncate=5, return_k_alternatives=3, best_of=1)
    Parameters(best_of=2, do_sample=True)
    Parameters(best_of=2, temperature=0.5)
    Parameters(temperature=0.0)                                        # zero temperature = greedy, accepted
    _bad(best_of=0)
    _bad(best_of=2)                                                    # needs sampling
    _bad(best_of=2, do_sample=True, seed=1)                            # seed and best_of > 1 exclude each other
    _bad(repetition_penalty=0.0)
    _bad(frequency_penalty=2.5)
    _bad(presence_penalty=-2.5)
    _bad(seed=-1)
    _bad(temperature=-1.0)
    _bad(top_k=0)
    _bad(top_p=0.0)
    _bad(top_p=1.5)
    _bad(truncate=0)
    _bad(typical_p=1.0)
    _bad(typical_p=0.0)
    _bad(return_k_alternatives=0)
    _bad(adapter_source="ftp")
    _bad(adapter_id="x", merged_adapters=MergedAdapters(ids=["a"], weights=[1.0]))


def test_merged_adapters_and_request_rules():
    MergedAdapters(ids=["a", "b"], weights=[0.5, 0.5], merge_strategy="ties", density=0.3, majority_sign_method="frequency")
    for kw in (dict(ids=["a"], weights=[1.0, 2.0]), dict(ids=[], weights=[]), dict(ids=["a"], weights=[1.0], merge_strategy="average"),
               dict(ids=["a"], weights=[1.0], density=1.5), dict(ids=["a"], weights=[1.0], majority_sign_method="median")):
        with pytest.raises(Exception):
            MergedAdapters(**kw)
    Request(inputs="hello")
    Request(inputs="hello", parameters=Parameters(best_of=2, do_sample=True))
    with pytest.raises(Exception):
        Request(inputs="")
    with pytest.raises(Exception):
        Request(inputs="x", stream=True, parameters=Parameters(best_of=2, do_sample=True))
    rf = ResponseFormat(type=ResponseFormatType.json_object, schema_={"type": "object"})
    assert rf.to_dict() == {"type": "json_object", "schema": {"type": "object"}}
    assert ResponseFormat(type="text").to_dict() == {"type": "text"}


@pytest.mark.parametrize("status,payload,exc", [
    (424, {"error": "boom", "error_type": "generation"}, errors.GenerationError),
    (500, {"error": "cut", "error_type": "incomplete_generation"}, errors.IncompleteGenerationError),
    (429, {"error": "busy", "error_type": "overloaded"}, errors.OverloadedError),
    (422, {"error": "bad", "error_type": "validation"}, errors.ValidationError),
    (400, {"error": "bad request"}, errors.BadRequestError),
    (403, {"error": "loading"}, errors.ShardNotReadyError),
    (424, {"error": "loading"}, errors.ShardNotReadyError),
    (504, {"error": "slow"}, errors.ShardTimeoutError),
    (404, {"error": "nope"}, errors.NotFoundError),
    (429, {"error": "rate"}, errors.RateLimitExceededError),
    (500, {"error": "?"}, errors.UnknownError),
])
def test_error_mapping(status, payload, exc):
    e = errors.parse_error(status, payload)
    assert type(e) is exc and str(e) == payload["error"]


def test_response_format_takes_the_schema_under_its_public_name():
    """`ResponseFormat(type=..., schema=...)` is how callers of the reference client pass a JSON schema; the schema must reach the
    request body under `schema` whichever spelling built the object."""
    from lorax_b200.client import BatchRequest, DeployedModel
    from lorax_b200.client.types import Parameters, ResponseFormat
    schema = {"type": "object", "properties": {"a": {"type": "integer"}}}
    for fmt in (ResponseFormat(type="json_object", schema=schema), ResponseFormat(type="json_object", schema_=schema),
                ResponseFormat(type="json_object", schema_spec=schema), {"type": "json_object", "schema": schema}):
        body = Parameters(response_format=fmt).model_dump(by_alias=True, exclude_none=True)
        assert body["response_format"] == {"type": "json_object", "schema": schema}
    assert ResponseFormat(type="json_object", schema=schema).schema_spec == schema
    assert BatchRequest(inputs=["a", "b"]).stream is False and DeployedModel(model_id="m", sha="0").sha == "0"
    import pytest
    with pytest.raises(ValueError, match="cannot be empty"):
        BatchRequest(inputs=[])
