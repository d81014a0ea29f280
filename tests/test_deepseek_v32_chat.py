"""Prompt rendering and answer parsing of DeepSeek-V3.2's chat format (no Jinja template ships with the model).
Expected strings are written out by hand from the format's rules."""
import json

import pytest

from lightllm_b200.models import deepseek_v32_chat as v32

B, E, U, A = v32.BOS, v32.EOS, v32.USER_TAG, v32.ASSISTANT_TAG
D = v32.DSML

WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "weather of a city",
                                            "parameters": {"type": "object",
                                                           "properties": {"city": {"type": "string"},
                                                                          "days": {"type": "integer"}}}}}
CALL = {"type": "function", "function": {"name": "get_weather",
                                         "arguments": json.dumps({"city": "München", "days": 3, "units": ["C"]})}}
CALL_TEXT = (f'\n\n<{D}function_calls>\n<{D}invoke name="get_weather">\n'
             f'<{D}parameter name="city" string="true">München</{D}parameter>\n'
             f'<{D}parameter name="days" string="false">3</{D}parameter>\n'
             f'<{D}parameter name="units" string="false">["C"]</{D}parameter>\n'
             f'</{D}invoke>\n</{D}function_calls>')


def test_plain_chat_and_thinking_turns():
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"},
            {"role": "assistant", "content": "Hello!", "reasoning": "greet back"},
            {"role": "user", "content": "And now?"}]
    assert v32.render(msgs, thinking=False) == f"{B}Be brief.{U}Hi{A}</think>Hello!{E}{U}And now?{A}</think>"
    # thinking mode: only the last user turn opens a think block; older reasoning is not fed back
    assert v32.render(msgs, thinking=True) == f"{B}Be brief.{U}Hi{A}</think>Hello!{E}{U}And now?{A}<think>"
    # continuing a rendered context: no BOS, only the new messages
    assert v32.render(msgs[3:], thinking=True, context=msgs[:3]) == f"{U}And now?{A}<think>"
    assert v32.render(msgs[:2], add_bos=False) == f"Be brief.{U}Hi{A}</think>"


def test_tools_calls_and_results():
    msgs = [{"role": "system", "content": "sys", "tools": [WEATHER]},
            {"role": "user", "content": "weather?"},
            {"role": "assistant", "content": "", "reasoning": "need the tool", "tool_calls": [CALL, CALL]},
            {"role": "tool", "content": "sunny"}, {"role": "tool", "content": "rain"}]
    out = v32.render(msgs, thinking=True)
    sys_part = "sys\n\n" + v32.tools_section([WEATHER])
    assert json.dumps(WEATHER["function"], ensure_ascii=False) in sys_part and "<functions>\n" in sys_part
    two_calls = CALL_TEXT.replace(f"\n</{D}function_calls>", "") + CALL_TEXT.split(f"<{D}function_calls>")[1]
    expect = (f"{B}{sys_part}{U}weather?{A}<think>need the tool</think>{two_calls}{E}"
              "\n\n<function_results>\n<result>sunny</result>\n<result>rain</result>\n</function_results>\n\n<think>")
    assert out == expect
    # chat mode closes the think block after the results instead
    assert v32.render(msgs, thinking=False).endswith("</function_results>\n\n</think>")
    with pytest.raises(ValueError):
        v32.render(msgs + [{"role": "tool", "content": "one too many"}])
    with pytest.raises(ValueError):
        v32.render([{"role": "tool", "content": "orphan"}])
    with pytest.raises(ValueError):
        v32.render([{"role": "wizard", "content": "?"}])
    with pytest.raises(ValueError):   # thinking mode: an answer after the last user turn needs reasoning or calls
        v32.render([{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}], thinking=True)


def test_developer_prefix_and_response_format():
    msgs = [{"role": "developer", "content": "do it", "tools": [WEATHER], "response_format": {"type": "json_object"}},
            {"role": "assistant", "content": "{\"a\":", "prefix": True}]
    out = v32.render(msgs)
    assert out.startswith(f"{B}{U}\n\n## Tools\n")
    assert '## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n{"type": "json_object"}' in out
    assert out.endswith(f"\n\n# The user's message is: do it{A}</think>" + '{"a":')   # the prefix stays open
    # an older developer message is left out in thinking mode, like the published encoder does
    older = [{"role": "developer", "content": "old"}, {"role": "assistant", "content": "x"},
             {"role": "user", "content": "new"}]
    with_dev = v32.render(older, thinking=False)
    assert "old" in with_dev
    dropped = v32._without_old_reasoning(older)
    assert [m["role"] for m in dropped] == ["assistant", "user"]


def test_parse_completion_round_trip():
    answer = {"role": "assistant", "content": "It is sunny.", "reasoning": "look it up", "tool_calls": [CALL]}
    text = v32.render([{"role": "user", "content": "q"}, answer], thinking=True, add_bos=False)
    completion = text.split(A + "<think>", 1)[1]
    got = v32.parse_completion(completion, thinking=True)
    assert got["content"] == "It is sunny." and got["reasoning"] == "look it up"
    assert len(got["tool_calls"]) == 1 and got["tool_calls"][0]["function"]["name"] == "get_weather"
    assert json.loads(got["tool_calls"][0]["function"]["arguments"]) == {"city": "München", "days": 3, "units": ["C"]}
    plain = v32.parse_completion("Just text." + E)
    assert plain == {"role": "assistant", "content": "Just text.", "reasoning": "", "tool_calls": []}
    # a string parameter that looks like JSON stays a string
    weird = (f'ok\n\n<{D}function_calls>\n<{D}invoke name="f">\n<{D}parameter name="x" string="true">[1, 2]'
             f'</{D}parameter>\n</{D}invoke>\n</{D}function_calls>')
    assert json.loads(v32.parse_completion(weird)["tool_calls"][0]["function"]["arguments"]) == {"x": "[1, 2]"}
    for bad in ["no end token", "a" + E + "b", f"x\n\n<{D}function_calls>\n<{D}invoke name=\"f\">\n" + E,
                f"x\n\n<{D}function_calls>\nnoise</{D}function_calls>" + E, "nested <think> marker" + E]:
        with pytest.raises(ValueError):
            v32.parse_completion(bad)
    with pytest.raises(ValueError):
        v32.parse_completion("never closes its thoughts" + E, thinking=True)


class _Tok:
    eos_token_id = 1

    def encode(self, text, add_special_tokens=True):
        assert add_special_tokens is False
        return [ord(c) for c in text]

    def get_added_vocab(self):
        return {"<x>": 7}

    def apply_chat_template(self, msgs, **kw):
        return "jinja:" + kw["chat_template"]

    def __len__(self):
        return 11


def test_tokenizer_wrapper():
    t = v32.DeepSeekV32Tokenizer(_Tok())
    assert t.eos_token_id == 1 and len(t) == 11 and t.get_added_vocab() == {"<x>": 7} and t.chat_template
    msgs = [{"role": "user", "content": "Hi"}]
    assert t.apply_chat_template(conversation=msgs) == f"{B}{U}Hi{A}</think>"
    assert t.apply_chat_template(messages=msgs, thinking=True) == f"{B}{U}Hi{A}<think>"
    assert t.apply_chat_template(msgs, enable_thinking=True, tokenize=True) == [ord(c) for c in f"{B}{U}Hi{A}<think>"]
    # tools go into the system message (one is made when there is none), bare function dicts are accepted
    with_tools = t.apply_chat_template(msgs, tools=[WEATHER["function"]])
    assert with_tools == B + "\n\n" + v32.tools_section([WEATHER]) + f"{U}Hi{A}</think>"
    assert msgs == [{"role": "user", "content": "Hi"}]     # the caller's list is untouched
    sys_msgs = [{"role": "system", "content": "S"}] + msgs
    assert t.apply_chat_template(sys_msgs, tools=[WEATHER]).startswith(B + "S\n\n## Tools\n")
    assert t.apply_chat_template(msgs, chat_template="T") == "jinja:T"


def test_factory_wraps_by_model_type(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from lightllm_b200.server.tokenizer import get_tokenizer

    tok = Tokenizer(models.WordLevel({"[UNK]": 0, "Hi": 1}, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="[UNK]").save_pretrained(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "deepseek_v32"}))
    t = get_tokenizer(str(tmp_path))
    assert isinstance(t, v32.DeepSeekV32Tokenizer)
    assert t.apply_chat_template([{"role": "user", "content": "Hi"}]) == f"{B}{U}Hi{A}</think>"
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama"}))
    assert not isinstance(get_tokenizer(str(tmp_path)), v32.DeepSeekV32Tokenizer)
