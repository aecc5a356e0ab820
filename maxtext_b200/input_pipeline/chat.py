"""Chat formatting for supervised fine-tuning and decoding (`use_chat_template`, `chat_template`, `chat_template_path`;
src/maxtext/input_pipeline/input_pipeline_utils.py, instruction_data_processing.py).

A conversation is a list of {"role", "content"} messages. The template is a Jinja2 string in the HuggingFace convention
(variables `messages`, `add_generation_prompt`, `bos_token`, `eos_token`); it comes from `chat_template`, from the
`chat_template` field of the JSON file named by `chat_template_path`, or falls back to a plain "role: content" layout.
For training the conversation is split at the last assistant turn: everything before it (rendered with the generation
prompt) is the prompt, the assistant's text is the completion, so completion-only masking applies to chat data too."""
from __future__ import annotations

import json

DEFAULT_TEMPLATE = (
    "{% for m in messages %}{{ m['role'] }}: {{ m['content'] }}\n{% endfor %}"
    "{% if add_generation_prompt %}assistant: {% endif %}")


def load_template(config) -> str:
  t = str(getattr(config, "chat_template", "") or "")
  path = str(getattr(config, "chat_template_path", "") or "")
  if not t and path:
    with open(path, "r", encoding="utf-8") as fh:
      data = json.load(fh)
    t = data.get("chat_template", "") if isinstance(data, dict) else str(data)
  return t or DEFAULT_TEMPLATE


def render(messages: list[dict], template: str, add_generation_prompt: bool = False, bos_token: str = "", eos_token: str = "") -> str:
  import jinja2
  env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False)
  return env.from_string(template).render(messages=messages, add_generation_prompt=add_generation_prompt, bos_token=bos_token,
                                          eos_token=eos_token)


def split_for_sft(messages: list[dict], template: str) -> tuple[str, str]:
  """(prompt text, completion text): the conversation up to the last assistant turn, and that turn's content."""
  last = max((i for i, m in enumerate(messages) if m.get("role") == "assistant"), default=None)
  if last is None:
    return render(messages, template, True), ""
  return render(messages[:last], template, True), str(messages[last].get("content", ""))
