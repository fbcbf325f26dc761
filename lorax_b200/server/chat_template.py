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


def render_chat(messages: List[dict], template: Optional[str], tools=None, bos_token: str = "", eos_token: str = "",
                add_generation_prompt: bool = True) -> str:
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(msg):
        raise TemplateError(msg)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    norm = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):       # OpenAI content parts -> text
            m["content"] = "".join(p.get("text", "") for p in c if isinstance(p, dict))
        norm.append(m)
    try:
        return env.from_string(template or DEFAULT_TEMPLATE).render(
            messages=norm, bos_token=bos_token, eos_token=eos_token, add_generation_prompt=add_generation_prompt,
            tools=tools, tools_in_user_message=False)
    except TemplateError:
        raise
    except Exception as e:
        raise TemplateError(str(e)) from e
