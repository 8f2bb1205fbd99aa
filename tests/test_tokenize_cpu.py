"""Tokenizer front end and Jinja chat templates (ferrotorch-tokenize/src/lib.rs)."""
import json

import pytest

from ferrotorch_b200.utils import text as T

LLAMA3_STYLE = ("{{ bos_token }}{% for message in messages %}{% if message['role'] not in ['system', 'user', 'assistant'] %}"
                "{{ raise_exception('unknown role ' + message['role']) }}{% endif %}"
                "{{ '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n' + message['content'] | trim + '<|eot_id|>' }}"
                "{% endfor %}{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")
MSGS = [{"role": "system", "content": "be brief "}, {"role": "user", "content": "hi"}]


def _tokenizer(tmp_path):
    tk = pytest.importorskip("tokenizers")
    vocab = {w: i for i, w in enumerate(["[UNK]", "[BOS]", "hello", "world", "be", "brief", "hi", "user", "system"])}
    tok = tk.Tokenizer(tk.models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = tk.pre_tokenizers.Whitespace()
    p = tmp_path / "tokenizer.json"
    tok.save(str(p))
    return T.load_tokenizer(str(p))


def test_tokenizer_helpers(tmp_path):
    tok = _tokenizer(tmp_path)
    assert T.encode(tok, "hello world zzz") == [2, 3, 0] and T.decode(tok, [2, 3]) == "hello world"
    assert T.encode_batch(tok, ["hi", "be brief"]) == [[6], [4, 5]]
    assert T.vocab_size(tok) == 9 and T.token_to_id(tok, "hi") == 6 and T.token_to_id(tok, "nope") is None
    assert T.id_to_token(tok, 3) == "world" and T.id_to_token(tok, 99) is None
    with pytest.raises(Exception):
        T.load_tokenizer(str(tmp_path / "missing.json"))


def test_jinja_chat_templates(tmp_path):
    out = T.apply_chat_template(MSGS, LLAMA3_STYLE, True, bos_token="<|begin_of_text|>")
    assert out == ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nbe brief<|eot_id|>"
                   "<|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    assert T.apply_chat_template([{"role": "system", "content": "be brief"}, T.ChatMessage("user", "hi")]) == out  # built-in layout
    assert T.apply_chat_template(MSGS, LLAMA3_STYLE, False).endswith("hi<|eot_id|>")
    assert T.apply_chat_template(MSGS, "chatml", True) == \
        "<|im_start|>system\nbe brief <|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    with pytest.raises(ValueError, match="unknown role tool"):
        T.apply_chat_template([{"role": "tool", "content": "x"}], LLAMA3_STYLE)
    with pytest.raises(ValueError, match="invalid chat template"):
        T.apply_chat_template(MSGS, "{% for %}")
    # extra fields are visible to the template; strftime_now is a function of the environment
    m = T.ChatMessage("user", "hi", {"name": "ann"})
    assert T.apply_chat_template([m], "{{ messages[0].name }}:{{ messages[0].content }}{{ eos_token }}", eos_token="</s>") == "ann:hi</s>"
    assert len(T.apply_chat_template([], "{{ strftime_now('%Y') }}")) == 4
    # the sandbox keeps templates away from Python internals
    with pytest.raises(ValueError):
        T.apply_chat_template(MSGS, "{{ messages.__class__.__mro__ }}")
    tok = _tokenizer(tmp_path)
    prompt, ids = T.apply_chat_template_to_ids(tok, "{% for m in messages %}{{ m.role }} {{ m.content }} {% endfor %}", MSGS)
    assert prompt == "system be brief  user hi " and ids == [8, 4, 5, 7, 6]


def test_chat_template_agrees_with_transformers(tmp_path):
    tr = pytest.importorskip("transformers")
    tok = _tokenizer(tmp_path)
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="[BOS]")
    want = fast.apply_chat_template(MSGS, chat_template=LLAMA3_STYLE, tokenize=False, add_generation_prompt=True)
    assert T.apply_chat_template(MSGS, LLAMA3_STYLE, True, bos_token="[BOS]") == want


def test_load_chat_template(tmp_path):
    p = tmp_path / "tokenizer_config.json"
    p.write_text(json.dumps({"chat_template": "{{ bos_token }}x"}))
    assert T.load_chat_template(str(p)) == "{{ bos_token }}x"
    p.write_text(json.dumps({"chat_template": [{"name": "default", "template": "A"}, {"name": "tool_use", "template": "B"}]}))
    assert T.load_chat_template(str(p)) == "A"
    p.write_text(json.dumps({"model_max_length": 8}))
    assert T.load_chat_template(str(p)) is None
    p.write_text(json.dumps({"chat_template": 7}))
    with pytest.raises(ValueError, match="unexpected type"):
        T.load_chat_template(str(p))
    p.write_text("{oops")
    with pytest.raises(ValueError, match="parse"):
        T.load_chat_template(str(p))
    with pytest.raises(OSError):
        T.load_chat_template(str(tmp_path / "none.json"))
