"""Chat template rendering (Jinja2, sandboxed), the part of the router that the reference does with minijinja
(`router/src/infer.rs:40-147`): `messages`, `bos_token`, `eos_token`, `add_generation_prompt`, `tools`,
`raise_exception` and `strftime_now` are available to the template."""

from __future__ import annotations

import datetime
from typing import List, Optional

DEFAULT_TEMPLATE = (
    "{% for message in messages %}{{ '<|' + message['role'] + '|>\\n' + message['content'] + '\\n' }}{% endfor %}"
    "{% if add_generation_prompt %}{{ '<|assistant|>\\n' }}{% endif %}"
)


class TemplateError(ValueError):
    pass


DEFAULT_TOOL_PROMPT = ("\nGiven the functions available, please respond with a JSON for a function call with its proper arguments that "
                       "best answers the given prompt. Respond in the format {name: function name, parameters: dictionary of argument "
                       "name and its value}.Do not use variables.\n")


def render_chat(messages: List[dict], template: Optional[str], tools=None, bos_token: str = "", eos_token: str = "",
                add_generation_prompt: bool = True, guideline: Optional[str] = None, tool_prompt: Optional[str] = None) -> str:
    """Prompt text of a chat request.  As in the reference (`router/src/infer.rs:97-147`): a template that names `guideline`
    needs one; with tools, the tool prompt is appended to the last message, preceded by the tools as JSON when the template
    itself has no place for them."""
    import json

    from jinja2 import meta
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(msg):
        raise TemplateError(msg)

    # `break` / `continue` in loops: transformers renders chat templates with this extension on
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    source = template or DEFAULT_TEMPLATE
    try:
        variables = meta.find_undeclared_variables(env.parse(source))
    except Exception as e:
        raise TemplateError(str(e)) from e
    if "guideline" in variables and guideline is None:
        raise TemplateError("Missing template vatiable: guideline")
    norm = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):       # OpenAI content parts -> text
            m["content"] = "".join(p.get("text", "") for p in c if isinstance(p, dict))
        norm.append(m)
    if tools:
        prompt = DEFAULT_TOOL_PROMPT if tool_prompt is None else tool_prompt
        text = f"\n---\n{prompt}" if "tools" in variables else f"\n---\n{json.dumps(tools, separators=(',', ':'))}\n{prompt}"
        if norm:
            norm[-1]["content"] = (norm[-1].get("content") or "") + text
    try:
        return env.from_string(source).render(
            messages=norm, bos_token=bos_token, eos_token=eos_token, add_generation_prompt=add_generation_prompt,
            tools=tools or None, tools_in_user_message=False, guideline=guideline)
    except TemplateError:
        raise
    except Exception as e:
        raise TemplateError(str(e)) from e
