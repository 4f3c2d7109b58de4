"""Tools declared by decorating functions in a user's file, merged with the tools of a YAML file."""
import asyncio
import json

import pytest

from verl_b200.tools.function_tool import FUNCTION_TOOL_REGISTRY, function_tool, load_function_tools_from_path
from verl_b200.tools.registry import load_all_tools

SOURCE = '''
from verl_b200.tools.function_tool import function_tool


@function_tool
def add(a: int, b: int) -> int:
    """Add two integers.

    Args:
        a: first addend
        b: second addend
    """
    return a + b


@function_tool(name="shout", description="Upper-case a text.")
async def _shout(text: str):
    return text.upper()
'''


def test_functions_of_a_file_become_tools_once(tmp_path):
    path = tmp_path / "my_tools.py"
    path.write_text(SOURCE)
    tools = load_function_tools_from_path(str(path))
    assert [t.name for t in tools] == ["add", "shout"] and load_function_tools_from_path(str(path)) is tools   # loaded once
    add, shout = tools
    schema = add.tool_schema.model_dump(exclude_none=True)["function"]
    assert schema["name"] == "add" and set(schema["parameters"]["properties"]) == {"a", "b"} and schema["parameters"]["required"] == ["a", "b"]
    assert shout.tool_schema.function.description == "Upper-case a text."
    res, _, _ = asyncio.run(add.execute("i", {"a": 2, "b": 5}))
    assert json.loads(res.text) == 7
    res, _, _ = asyncio.run(shout.execute("i", {"text": "hi"}))
    assert res.text == "HI"
    res, _, info = asyncio.run(add.execute("i", {"a": 1}))      # an error is an observation for the model
    assert "Error when executing tool" in res.text and info == {"tool_error": 1}
    with pytest.raises(FileNotFoundError):
        load_function_tools_from_path(str(tmp_path / "absent.py"))
    for n in ("add", "shout"):
        FUNCTION_TOOL_REGISTRY.pop(n, None)


def test_variadic_parameters_duplicate_names_and_collisions_are_refused(tmp_path):
    with pytest.raises(ValueError, match="variadic"):
        @function_tool
        def bad(*args):
            return 0

    @function_tool(name="calc_once")
    def first(x: int):
        return x

    with pytest.raises(ValueError, match="already registered"):
        @function_tool(name="calc_once")
        def second(x: int):
            return x

    FUNCTION_TOOL_REGISTRY.pop("calc_once", None)
    py = tmp_path / "t.py"
    py.write_text("from verl_b200.tools.function_tool import function_tool\n\n@function_tool\ndef lookup(q: str):\n    return q\n")
    yml = tmp_path / "tools.yaml"
    yml.write_text("tools:\n- class_name: tests.test_function_tools_on_cpu.Lookup\n  config: {type: native}\n"
                   "  tool_schema: {type: function, function: {name: lookup, description: d, parameters: {type: object, properties: {}, required: []}}}\n")
    with pytest.raises(ValueError, match="collide"):
        load_all_tools(str(yml), str(py))
    assert [t.name for t in load_all_tools(None, str(py))] == ["lookup"] and load_all_tools(None, None) == []
    FUNCTION_TOOL_REGISTRY.pop("lookup", None)


from verl_b200.tools.base_tool import BaseTool  # noqa: E402


class Lookup(BaseTool):
    pass
