"""The router's chat template interpreter against Jinja2 (the shard's renderer, `lorax_b200.server.chat_template.render_chat`) on the
templates of well-known model families and on the constructs each alone.  The reference router renders chat templates itself
(minijinja, router/src/infer.rs:40-147)."""

import pytest

from lorax_b200.router.native import chat_render
from lorax_b200.server.chat_template import DEFAULT_TEMPLATE, TemplateError, render_chat

CHATML = ("{% for message in messages %}{{'<|im_start|>' + message['role'] + '\n' + message['content'] + '<|im_end|>' + '\n'}}{% endfor %}"
          "{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}")
LLAMA3 = ("{% set loop_messages = messages %}{% for message in loop_messages %}{% set content = '<|start_header_id|>' + message['role'] + "
          "'<|end_header_id|>\n\n'+ message['content'] | trim + '<|eot_id|>' %}{% if loop.index0 == 0 %}{% set content = bos_token + content %}"
          "{% endif %}{{ content }}{% endfor %}{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")
MISTRAL = ("{{ bos_token }}{% for message in messages %}{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}"
           "{{ raise_exception('Conversation roles must alternate user/assistant/user/assistant/...') }}{% endif %}"
           "{% if message['role'] == 'user' %}{{ '[INST] ' + message['content'] + ' [/INST]' }}{% elif message['role'] == 'assistant' %}"
           "{{ message['content'] + eos_token}}{% else %}{{ raise_exception('Only user and assistant roles are supported!') }}{% endif %}{% endfor %}")
LLAMA2 = ("{% if messages[0]['role'] == 'system' %}{% set loop_messages = messages[1:] %}{% set system_message = messages[0]['content'] %}"
          "{% else %}{% set loop_messages = messages %}{% set system_message = false %}{% endif %}{% for message in loop_messages %}"
          "{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}{{ raise_exception('Conversation roles must alternate') }}{% endif %}"
          "{% if loop.index0 == 0 and system_message != false %}{% set content = '<<SYS>>\\n' + system_message + '\\n<</SYS>>\\n\\n' + message['content'] %}"
          "{% else %}{% set content = message['content'] %}{% endif %}{% if message['role'] == 'user' %}{{ bos_token + '[INST] ' + content.strip() + ' [/INST]' }}"
          "{% elif message['role'] == 'assistant' %}{{ ' '  + content.strip() + ' ' + eos_token }}{% endif %}{% endfor %}")
ZEPHYR = ("{% for message in messages %}\n{% if message['role'] == 'user' %}\n{{ '<|user|>\n' + message['content'] + eos_token }}\n"
          "{% elif message['role'] == 'system' %}\n{{ '<|system|>\n' + message['content'] + eos_token }}\n{% elif message['role'] == 'assistant' %}\n"
          "{{ '<|assistant|>\n'  + message['content'] + eos_token }}\n{% endif %}\n{% if loop.last and add_generation_prompt %}\n{{ '<|assistant|>' }}\n"
          "{% endif %}\n{% endfor %}")
GEMMA = ("{{ bos_token }}{% if messages[0]['role'] == 'system' %}{{ raise_exception('System role not supported') }}{% endif %}"
         "{% for message in messages %}{% if (message['role'] == 'user') != (loop.index0 % 2 == 0) %}{{ raise_exception('Conversation roles must alternate') }}"
         "{% endif %}{% if (message['role'] == 'assistant') %}{% set role = 'model' %}{% else %}{% set role = message['role'] %}{% endif %}"
         "{{ '<start_of_turn>' + role + '\n' + message['content'] | trim + '<end_of_turn>\n' }}{% endfor %}"
         "{% if add_generation_prompt %}{{'<start_of_turn>model\n'}}{% endif %}")
PHI3 = ("{% for message in messages %}{% if message['role'] == 'system' %}{{'<|system|>\n' + message['content'] + '<|end|>\n'}}"
        "{% elif message['role'] == 'user' %}{{'<|user|>\n' + message['content'] + '<|end|>\n'}}{% elif message['role'] == 'assistant' %}"
        "{{'<|assistant|>\n' + message['content'] + '<|end|>\n'}}{% endif %}{% endfor %}{% if add_generation_prompt %}{{ '<|assistant|>\n' }}"
        "{% else %}{{ eos_token }}{% endif %}")
QWEN_TOOLS = """{%- if tools %}
    {{- '<|im_start|>system\\n' }}
    {%- if messages[0]['role'] == 'system' %}
        {{- messages[0]['content'] }}
    {%- else %}
        {{- 'You are a helpful assistant.' }}
    {%- endif %}
    {{- "\\n\\n# Tools\\n\\nYou may call one or more functions.\\n<tools>" }}
    {%- for tool in tools %}
        {{- "\\n" }}
        {{- tool | tojson }}
    {%- endfor %}
    {{- "\\n</tools><|im_end|>\\n" }}
{%- else %}
    {%- if messages[0]['role'] == 'system' %}
        {{- '<|im_start|>system\\n' + messages[0]['content'] + '<|im_end|>\\n' }}
    {%- endif %}
{%- endif %}
{%- for message in messages %}
    {%- if (message.role == "user") or (message.role == "system" and not loop.first) or (message.role == "assistant" and not message.tool_calls) %}
        {{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>' + '\\n' }}
    {%- elif message.role == "assistant" %}
        {{- '<|im_start|>' + message.role }}
        {%- if message.content %}
            {{- '\\n' + message.content }}
        {%- endif %}
        {%- for tool_call in message.tool_calls %}
            {%- if tool_call.function is defined %}
                {%- set tool_call = tool_call.function %}
            {%- endif %}
            {{- '\\n<tool_call>\\n{"name": "' }}
            {{- tool_call.name }}
            {{- '", "arguments": ' }}
            {{- tool_call.arguments | tojson }}
            {{- '}\\n</tool_call>' }}
        {%- endfor %}
        {{- '<|im_end|>\\n' }}
    {%- elif message.role == "tool" %}
        {%- if (loop.index0 == 0) or (messages[loop.index0 - 1].role != "tool") %}
            {{- '<|im_start|>user' }}
        {%- endif %}
        {{- '\\n<tool_response>\\n' }}
        {{- message.content }}
        {{- '\\n</tool_response>' }}
        {%- if loop.last or (messages[loop.index0 + 1].role != "tool") %}
            {{- '<|im_end|>\\n' }}
        {%- endif %}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|im_start|>assistant\\n' }}
{%- endif %}
"""
NAMESPACE = """{% set ns = namespace(system='', n=0) %}
{% for m in messages %}
  {% if m.role == 'system' %}{% set ns.system = ns.system ~ m.content %}{% else %}{% set ns.n = ns.n + 1 %}{% endif %}
{% endfor %}
{# a comment #}
{{ ns.system | upper }}|{{ ns.n }}|{{ messages | length }}|{{ messages[-1]['content'][:5] }}|{{ 'yes' if ns.n > 1 else 'no' }}
{% for m in messages if m.role != 'system' %}{{ loop.index }}/{{ loop.length }}:{{ m.content | default('none') | replace('a', 'A') }}{{ ', ' if not loop.last }}{% else %}empty{% endfor %}
{% for k, v in {'b': 1, 'a': [1, 2.5, true, none, 'x']}.items() %}{{ k }}={{ v | tojson }};{% endfor %}
{{ [1, 2, 3] | join('-') }} {{ 'a,b' .split(',') | last }} {{ 7 // 2 }} {{ 7 % 3 }} {{ 2 * 3.5 }} {{ 1 / 4 }} {{ 'x' in 'xyz' }} {{ 3 not in [1, 2] }} {{ none is none }} {{ undefined_thing is defined }}
{%- if messages[0].content.startswith('You') and messages[0].content is string %} starts{% endif %}
{{ "tab\\there" }}{{ '\\u00e9' }}{{ messages[0]['missing'] }}|{{ {"k": "<v>"} | tojson }}|{{ "Title me" | title }}|{{ range(3) | list }}
"""

MISTRAL_V3 = """{{- bos_token }}
{%- set user_messages = messages | selectattr('role', 'equalto', 'user') | list %}
{%- for message in messages %}
    {%- if message['role'] == 'user' %}
        {%- if tools and (message == user_messages[-1]) %}
            {{- ' [AVAILABLE_TOOLS] ' }}{{ tools | map(attribute='function') | map(attribute='name') | join(', ') }}{{ tools[0].function.parameters.properties | dictsort | tojson }}{{- ' [/AVAILABLE_TOOLS]' }}
        {%- endif %}
        {{- ' [INST] ' + message['content'] + ' [/INST]' }}
    {%- elif message['role'] == 'assistant' %}
        {{- ' ' + message['content'] + eos_token }}
    {%- else %}
        {{- '(' ~ message.role ~ ')' ~ message.content | indent(2) }}
    {%- endif %}
{%- endfor %}
{{- messages | rejectattr('role', 'in', ['user', 'system']) | map(attribute='content') | map('upper') | list | tojson }}
{{- [3, 1, 2] | max }}{{ [3, 1.5] | sum }}{{ ['b', 'a', 'b'] | unique | join }}{{ messages | map(attribute='nope', default='-') | join }}"""
LLAMA31 = """{{- bos_token }}
{%- if custom_tools is defined %}
    {%- set tools = custom_tools %}
{%- endif %}
{%- if not tools_in_user_message is defined %}
    {%- set tools_in_user_message = true %}
{%- endif %}
{%- if not date_string is defined %}
    {%- set date_string = "26 Jul 2024" %}
{%- endif %}
{%- if not tools is defined %}
    {%- set tools = none %}
{%- endif %}
{#- This block extracts the system message, so we can slot it into the right place. #}
{%- if messages[0]['role'] == 'system' %}
    {%- set system_message = messages[0]['content']|trim %}
    {%- set messages = messages[1:] %}
{%- else %}
    {%- set system_message = "" %}
{%- endif %}
{{- "<|start_header_id|>system<|end_header_id|>\n\n" }}
{%- if tools is not none %}
    {{- "Environment: ipython\n" }}
{%- endif %}
{{- "Cutting Knowledge Date: December 2023\n" }}
{{- "Today Date: " + date_string + "\n\n" }}
{%- if tools is not none and not tools_in_user_message %}
    {{- "You have access to the following functions." }}
    {%- for t in tools %}
        {{- t | tojson(indent=4) }}
        {{- "\n\n" }}
    {%- endfor %}
{%- endif %}
{{- system_message }}
{{- "<|eot_id|>" }}
{%- for message in messages %}
    {%- if not (message.role == 'ipython' or message.role == 'tool' or 'tool_calls' in message) %}
        {{- '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n'+ message['content'] | trim + '<|eot_id|>' }}
    {%- elif 'tool_calls' in message %}
        {%- if not message.tool_calls|length == 1 %}
            {{- raise_exception("This model only supports single tool-calls at once!") }}
        {%- endif %}
        {%- set tool_call = message.tool_calls[0].function %}
        {{- '<|start_header_id|>assistant<|end_header_id|>\n\n' -}}
        {{- '{"name": "' + tool_call.name + '", ' }}
        {{- '"parameters": ' }}
        {{- tool_call.arguments | tojson }}
        {{- "}" }}
        {%- for arg_name, arg_val in tool_call.arguments | items %}
            {{- arg_name ~ '="' ~ arg_val ~ '"' }}
            {%- if not loop.last %}, {% endif %}
        {%- endfor %}
        {{- "<|eot_id|>" }}
    {%- elif message.role == "tool" or message.role == "ipython" %}
        {{- "<|start_header_id|>ipython<|end_header_id|>\n\n" }}
        {%- if message.content is mapping or message.content is iterable %}
            {{- message.content | tojson }}
        {%- else %}
            {{- message.content }}
        {%- endif %}
        {{- "<|eot_id|>" }}
    {%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|start_header_id|>assistant<|end_header_id|>\n\n' }}
{%- endif %}
"""

HERMES_MACRO = """{%- macro json_to_python_type(json_spec) %}
{%- set basic_type_map = {"string": "str", "number": "float", "integer": "int", "boolean": "bool"} %}
{%- if basic_type_map[json_spec.type] is defined %}
    {{- basic_type_map[json_spec.type] }}
{%- elif json_spec.type == "array" %}
    {{- "list[" +  json_to_python_type(json_spec|items) + "]"}}
{%- elif json_spec.type == "object" %}
    {%- if json_spec.additionalProperties is defined %}
        {{- "dict[str, " + json_to_python_type(json_spec.additionalProperties) + ']'}}
    {%- else %}
        {{- "dict" }}
    {%- endif %}
{%- else %}
    {{- "Any" }}
{%- endif %}
{%- endmacro %}
{%- macro greet(name, punct='!') %}Hello {{ name }}{{ punct }}{% endmacro %}
{{- bos_token }}
{%- for tool in tools or [] %}
    {{- tool.function.name + "(" }}
    {%- for param_name, param_fields in tool.function.parameters.properties|items %}
        {{- param_name + ": " + json_to_python_type(param_fields) }}
        {%- if not loop.last %}{{ ", " }}{% endif %}
    {%- endfor %}
    {{- ") -> " + json_to_python_type({"type": "object", "additionalProperties": {"type": "number"}}) + "\n" }}
{%- endfor %}
{%- for message in messages %}{{ greet(message.role) }}{{ greet(name=message.role, punct='?') }} {{ message.content }}
{% endfor %}"""

MESSAGES = [
    [{"role": "user", "content": "Hello there"}],
    [{"role": "system", "content": "You are a pirate. "}, {"role": "user", "content": "  What is 2+2?  "}, {"role": "assistant", "content": "Four, arr."},
     {"role": "user", "content": "And naïve café 日本語 <tags> & 'quotes'?"}],
    [{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}, {"role": "user", "content": [{"type": "text", "text": "part one "}, {"type": "text", "text": "part two"}]}],
]
TEMPLATES = {"default": DEFAULT_TEMPLATE, "chatml": CHATML, "llama3": LLAMA3, "mistral": MISTRAL, "llama2": LLAMA2, "zephyr": ZEPHYR, "gemma": GEMMA,
             "phi3": PHI3, "qwen_tools": QWEN_TOOLS, "namespace": NAMESPACE, "mistral_v3": MISTRAL_V3, "llama31": LLAMA31, "hermes_macro": HERMES_MACRO}
TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "Weather for a city <now> & 'later' é",
                                            "parameters": {"type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}}]


def both(template, messages, **kw):
    try:
        want = ("text", render_chat(messages, template, bos_token="<s>", eos_token="</s>", **kw))
    except TemplateError as e:
        want = ("error", str(e))
    got = chat_render(template, messages, bos_token="<s>", eos_token="</s>", **kw)
    return want, got


@pytest.mark.parametrize("name", sorted(TEMPLATES))
def test_templates_of_known_families_render_like_jinja2(name):
    for messages in MESSAGES:
        want, got = both(TEMPLATES[name], messages)
        assert "unsupported" not in got, (name, got)
        if want[0] == "text":
            assert got.get("text") == want[1], (name, messages, got)
        else:
            assert "error" in got, (name, messages, got)
            if "raise_exception" in TEMPLATES[name]:
                assert got["error"] == want[1]


def test_tools_go_into_the_template_or_into_the_last_message():
    for name in ("qwen_tools", "chatml", "llama3", "mistral_v3", "llama31", "hermes_macro"):
        for extra in ({}, {"tool_prompt": "\nUse the tools.\n"}):
            want, got = both(TEMPLATES[name], MESSAGES[1], tools=TOOLS, **extra)
            assert got.get("text") == want[1], (name, got)
    tool_turns = [{"role": "user", "content": "weather in Paris?"},
                  {"role": "assistant", "content": "", "tool_calls": [{"type": "function", "function": {"name": "get_weather", "arguments": {"city": "Paris", "days": 2}}}]},
                  {"role": "tool", "content": "{\"temp\": 21.5}"}, {"role": "tool", "content": "{\"temp\": 19}"}, {"role": "user", "content": "thanks"}]
    for t in (QWEN_TOOLS, LLAMA31):
        want, got = both(t, tool_turns, tools=TOOLS)
        assert got.get("text") == want[1], got


def test_guideline_and_whitespace_control():
    t = "{% if guideline %}G:{{ guideline }}\n{% endif %}   {%- for m in messages %}\n  {% if true %}\n  x{{ m.content }}  \n  {%+ endif %}\n{% endfor -%}\n\n  end"
    want, got = both(t, MESSAGES[0], guideline="be nice")
    assert got.get("text") == want[1], (got, want)
    want, got = both(t, MESSAGES[0])
    assert want[0] == "error" and "error" in got and "guideline" in got["error"]
    for t in ["{% set block %}\n  <{{ messages | length }}>\n{% endset %}{{ block | trim }}{% for m in messages %}{{ loop.cycle('a', 'b', 'c') }}{% endfor %}",
              "{% for m in messages %}{% if m.role == 'system' %}{% continue %}{% endif %}{{ m.role }};{% if loop.index == 3 %}{% break %}{% endif %}{% endfor %}|"
              "{% for i in range(5) %}{% for j in range(5) %}{% if j > i %}{% break %}{% endif %}{{ j }}{% endfor %},{% endfor %}",
              "a\n  {# c #}\nb {{ 1 }}\n  {{ 2 }}\n{% set x = 3 %}\n{{ x }}\n", "{{- 'a' -}}  \n  b  {{- 'c' }}\n{%- if true -%}\n d \n{%- endif -%}\n e",
              "  {% if true %}  \n  {% endif %}  tail\n", "\t{%+ if true %}\tkept{% endif +%}\nnext"]:
        want, got = both(t, MESSAGES[1])
        assert got.get("text") == want[1], (t, got, want)


def test_what_the_interpreter_does_not_implement_is_reported_as_such():
    for t in ["{{ messages | groupby('role') | list }}", "{% filter upper %}a{% endfilter %}",
"{% call f() %}x{% endcall %}", "{{ '%s!' % messages[0].role }}", "{{ 'a{}'.format(1) }}", "{% set a, b = 1, 2 %}{{ a }}",
              "{% for m in messages recursive %}{{ m.role }}{% endfor %}", "{{ messages[::-1] | length }}"]:
        got = chat_render(t, MESSAGES[1])
        assert "unsupported" in got, (t, got)
    got = chat_render("{{ 'a' + 1 }}", MESSAGES[0])
    assert "error" in got
    got = chat_render("{{ messages[0].content.nope.deeper }}", MESSAGES[0])
    assert "error" in got
