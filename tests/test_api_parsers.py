"""Tool-call detectors, the streaming tool parser, the reasoning parser and the partial-JSON reader.
Scenarios follow the reference's parser tests (xllm/function_call/*_test.cpp, xllm/parser/reasoning_parser_test.cpp):
single / multiple calls, text before the call, calls streamed in arbitrary chunk sizes, malformed sections."""
import json

import pytest

from xllm_wxh_b200.api.function_call import StreamingToolParser, parse_tool_calls, resolve_parser
from xllm_wxh_b200.api.partial_json import parse_partial
from xllm_wxh_b200.api.reasoning_parser import ReasoningParser, resolve_reasoning_parser

ARGS1 = {"location": "Beijing", "unit": "celsius", "days": 3}
ARGS2 = {"query": "a \"quoted\" {brace}", "n": [1, 2, {"k": None}]}


def _sample(parser):
    a1, a2 = json.dumps(ARGS1, ensure_ascii=False), json.dumps(ARGS2, ensure_ascii=False)
    if parser == "qwen25":
        return ("Let me check.\n<tool_call>\n{\"name\": \"get_weather\", \"arguments\": " + a1 + "}\n</tool_call>\n"
                "<tool_call>\n{\"name\": \"search\", \"arguments\": " + a2 + "}\n</tool_call>")
    if parser == "kimi_k2":
        return ("Let me check.<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>" + a1 +
                "<|tool_call_end|><|tool_call_begin|>functions.search:1<|tool_call_argument_begin|>" + a2 +
                "<|tool_call_end|><|tool_calls_section_end|>")
    if parser == "deepseekv3":
        return ("Let me check.<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n" + a1 +
                "\n```<｜tool▁call▁end｜>\n<｜tool▁call▁begin｜>function<｜tool▁sep｜>search\n```json\n" + a2 +
                "\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>")
    raise KeyError(parser)


@pytest.mark.parametrize("parser", ["qwen25", "kimi_k2", "deepseekv3"])
def test_json_style_detectors_full_text(parser):
    text, calls = parse_tool_calls(_sample(parser), parser)
    assert text.strip() == "Let me check."
    assert [c.name for c in calls] == ["get_weather", "search"]
    assert json.loads(calls[0].arguments) == ARGS1
    assert json.loads(calls[1].arguments) == ARGS2
    assert calls[0].id and calls[0].id != calls[1].id


@pytest.mark.parametrize("parser", ["qwen25", "kimi_k2", "deepseekv3"])
@pytest.mark.parametrize("chunk", [1, 3, 7, 1000])
def test_json_style_detectors_streaming(parser, chunk):
    full = _sample(parser)
    sp = StreamingToolParser(parser)
    text, names, args, ids = "", {}, {}, {}
    for i in range(0, len(full), chunk):
        t, deltas = sp.feed(full[i:i + chunk])
        text += t
        for d in deltas:
            if d.name is not None:
                assert d.index not in names, "a call's name is sent once"
                names[d.index] = d.name
                ids[d.index] = d.id
            args[d.index] = args.get(d.index, "") + d.arguments
    text += sp.flush()
    assert text.strip() == "Let me check."
    assert names == {0: "get_weather", 1: "search"}
    assert json.loads(args[0]) == ARGS1 and json.loads(args[1]) == ARGS2
    assert ids[0] and ids[1] and ids[0] != ids[1]


def test_glm45_key_value_pairs():
    text = ("I will look.<tool_call>get_weather\n<arg_key>location</arg_key>\n<arg_value>Beijing</arg_value>\n"
            "<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>")
    rest, calls = parse_tool_calls(text, "glm45")
    assert rest.strip() == "I will look."
    assert calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"location": "Beijing", "days": 3}


def test_qwen3_coder_xml_parameters():
    text = ("<tool_call>\n<function=run>\n<parameter=cmd>\nls -la\n</parameter>\n<parameter=timeout>\n30\n</parameter>\n"
            "</function>\n</tool_call>")
    rest, calls = parse_tool_calls(text, "qwen3_coder")
    assert rest.strip() == ""
    assert calls[0].name == "run" and json.loads(calls[0].arguments) == {"cmd": "ls -la", "timeout": 30}


def test_plain_text_passes_through_and_marker_prefix_is_held_back():
    sp = StreamingToolParser("qwen25")
    t1, d1 = sp.feed("no tools here <tool")
    assert t1 == "no tools here " and not d1          # "<tool" could still become the marker
    t2, d2 = sp.feed("box>")
    assert t1 + t2 + sp.flush() == "no tools here <toolbox>" and not d2
    text, calls = parse_tool_calls("just an answer", "qwen25")
    assert text == "just an answer" and calls == []


def test_malformed_section_does_not_raise():
    text, calls = parse_tool_calls("x<tool_call>\n{\"name\": \"f\", \"arguments\": {\"a\": \n</tool_call>", "qwen25")
    assert calls == [] or calls[0].name == "f"


def test_resolve_auto():
    assert resolve_parser("auto", "qwen3") == "qwen25"
    assert resolve_parser("auto", "deepseek_v3") == "deepseekv3"
    assert resolve_parser("qwen3", "") == "qwen25"
    with pytest.raises(ValueError):
        resolve_parser("nope", "")
    assert resolve_reasoning_parser("auto", "qwen3") == "qwen3"


# ----------------------------------------------------------------------------- reasoning
def test_reasoning_full_text():
    r, c = ReasoningParser("qwen3").parse("<think>step 1\nstep 2</think>\n\nThe answer is 4.")
    assert r == "step 1\nstep 2" and c.strip() == "The answer is 4."
    r, c = ReasoningParser("qwen3").parse("No thinking at all.")
    assert r == "" and c == "No thinking at all."


def test_reasoning_forced_open_tag():
    """DeepSeek-R1 style templates open the think block in the prompt: the output starts inside it."""
    r, c = ReasoningParser("deepseek-r1").parse("chain of thought</think>final")
    assert r == "chain of thought" and c == "final"


@pytest.mark.parametrize("chunk", [1, 2, 5, 100])
def test_reasoning_streaming(chunk):
    full = "<think>alpha beta</think>gamma <b>delta</b>"
    rp = ReasoningParser("qwen3")
    r = c = ""
    for i in range(0, len(full), chunk):
        dr, dc = rp.feed(full[i:i + chunk])
        r, c = r + dr, c + dc
    dr, dc = rp.flush()
    r, c = r + dr, c + dc
    assert r == "alpha beta" and c == "gamma <b>delta</b>"


def test_reasoning_truncated_inside_think_block():
    rp = ReasoningParser("qwen3")
    r, c = rp.feed("<think>never clo")
    r2, c2 = rp.flush()
    assert (r + r2) == "never clo" and (c + c2) == ""


# ----------------------------------------------------------------------------- partial JSON
@pytest.mark.parametrize("text,want,complete", [
    ('{"a": 1, "b": [1, 2', {"a": 1, "b": [1, 2]}, False),
    ('{"a": "unterminated str', {"a": "unterminated str"}, False),
    ('{"a": 1, "b"', {"a": 1}, False),
    ('{"a": 1, "b":', {"a": 1}, False),
    ('{"a": {"x": tr', {"a": {}}, False),
    ('{"a": -1.5e', {"a": -1.5}, False),
    ('[{"k": "v"}, {"k2": "esc\\"aped', [{"k": "v"}, {"k2": 'esc"aped'}], False),
    ('{"done": true}', {"done": True}, True),
    ('', None, False),
])
def test_partial_json(text, want, complete):
    assert parse_partial(text) == (want, complete)


def test_partial_json_every_prefix_of_a_document_parses():
    doc = json.dumps({"name": "f", "arguments": {"s": "a\\b\"cé", "n": [1.5, -2, True, None], "o": {"p": {}}}})
    for i in range(1, len(doc) + 1):
        v, done = parse_partial(doc[:i])
        assert done == (i == len(doc))
    assert v == json.loads(doc)


# --- GLM-4.7 compact tags and DeepSeek-V3.2 DSML (the cases of the reference's glm47_detector_test.cpp / deepseekv32_detector_test.cpp)
def test_glm47_compact_format():
    text = ("Please help me check the weather <tool_call>get_weather<arg_key>city</arg_key><arg_value>北京</arg_value>"
            "<arg_key>date</arg_key><arg_value>2024-06-27</arg_value></tool_call>")
    rest, calls = parse_tool_calls(text, "glm47")
    assert rest == "Please help me check the weather" and len(calls) == 1 and calls[0].name == "get_weather"
    assert json.loads(calls[0].arguments) == {"city": "北京", "date": "2024-06-27"}
    rest, calls = parse_tool_calls("Calculate <tool_call>calculate<arg_key>expression</arg_key><arg_value>3.14 * 2</arg_value>"
                                   "<arg_key>precision</arg_key><arg_value>2</arg_value></tool_call>", "glm47")
    args = json.loads(calls[0].arguments)
    assert args == {"expression": "3.14 * 2", "precision": 2} and isinstance(args["precision"], int)
    # a block without arguments is not a call; an unfinished block is ignored; the line-broken GLM-4.5 form still parses
    assert parse_tool_calls("Test empty content <tool_call>test</tool_call>", "glm47")[1] == []
    assert parse_tool_calls("x <tool_call>get_weather<arg_key>city</arg_key><arg_value>a", "glm47")[1] == []
    _, calls = parse_tool_calls("<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n</tool_call>", "glm47")
    assert calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"city": "Paris"}
    assert resolve_parser("glm47") == "glm47" and resolve_parser("glm5") == "glm47"


def test_glm47_streaming_emits_name_then_arguments():
    sp = StreamingToolParser("glm47")
    text = "Hi <tool_call>get_weather<arg_key>city</arg_key><arg_value>Rome</arg_value></tool_call>"
    out, deltas = "", []
    for i in range(0, len(text), 5):
        t, d = sp.feed(text[i:i + 5])
        out += t
        deltas += d
    out += sp.flush()
    assert out.strip() == "Hi"
    names = [d.name for d in deltas if d.name]
    assert names == ["get_weather"]
    assert json.loads("".join(d.arguments for d in deltas)) == {"city": "Rome"}


DSML = ('Please help me check the weather <｜DSML｜function_calls>\n<｜DSML｜invoke name="get_weather">\n'
        '<｜DSML｜parameter name="city" string="true">北京</｜DSML｜parameter>\n'
        '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n'
        '<｜DSML｜invoke name="calculate">{"expression": "1+1"}</｜DSML｜invoke>\n</｜DSML｜function_calls>')


def test_deepseekv32_dsml_calls():
    rest, calls = parse_tool_calls(DSML, "deepseekv32")
    assert rest == "Please help me check the weather"
    assert [c.name for c in calls] == ["get_weather", "calculate"]
    assert json.loads(calls[0].arguments) == {"city": "北京", "days": 3}
    assert json.loads(calls[1].arguments) == {"expression": "1+1"}
    # unfinished invoke: no call, the text before the block stays
    rest, calls = parse_tool_calls('Incomplete tool call <｜DSML｜function_calls><｜DSML｜invoke name="get_weather"><｜DSML｜parameter name="city" string="true">北', "deepseekv32")
    assert rest == "Incomplete tool call" and calls == []
    assert resolve_parser("deepseekv32") == "deepseekv32" and resolve_parser("auto", "deepseek_v32") == "deepseekv32"


def test_deepseekv32_streaming():
    sp = StreamingToolParser("deepseekv32")
    out, deltas = "", []
    for i in range(0, len(DSML), 7):
        t, d = sp.feed(DSML[i:i + 7])
        out += t
        deltas += d
    out += sp.flush()
    assert out.strip() == "Please help me check the weather"
    assert [d.name for d in deltas if d.name] == ["get_weather", "calculate"]
    by_index = {}
    for d in deltas:
        by_index[d.index] = by_index.get(d.index, "") + d.arguments
    assert json.loads(by_index[0]) == {"city": "北京", "days": 3} and json.loads(by_index[1]) == {"expression": "1+1"}


def test_service_mailbox_delivers_everything_in_order():
    """Outputs cross from the engine's thread to the event loop through a mailbox with one wake-up per burst: nothing is
    lost or reordered when the producer keeps posting while the loop drains."""
    import asyncio
    import collections
    import threading
    from xllm_wxh_b200.api.openai_service import APIService
    svc = APIService.__new__(APIService)                 # the mailbox needs no engine
    svc._mail, svc._mail_scheduled = collections.deque(), False
    got = []
    wakeups = [0]
    loop = asyncio.new_event_loop()
    real = loop.call_soon_threadsafe

    def counting(fn, *a):
        wakeups[0] += 1
        return real(fn, *a)
    loop.call_soon_threadsafe = counting
    n = 20000

    def produce():
        for i in range(n):
            svc._post(loop, got.append, i)
        real(loop.stop) if False else None
    th = threading.Thread(target=produce)

    async def main():
        th.start()
        while len(got) < n:
            await asyncio.sleep(0.001)
    loop.run_until_complete(asyncio.wait_for(main(), 30))
    th.join()
    loop.close()
    assert got == list(range(n))
    assert 1 <= wakeups[0] < n                            # bursts share wake-ups
