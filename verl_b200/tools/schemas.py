"""Tool schemas (OpenAI function-calling shape). Parity target: ``verl/tools/schemas.py`` (127 lines)."""

from __future__ import annotations

import json
from typing import Any, Literal, Optional

from pydantic import BaseModel, Field

__all__ = ["OpenAIFunctionPropertySchema", "OpenAIFunctionParametersSchema", "OpenAIFunctionSchema",
           "OpenAIFunctionToolSchema", "OpenAIFunctionParsedSchema", "OpenAIFunctionCallSchema", "OpenAIFunctionToolCall",
           "ToolResponse"]


class OpenAIFunctionPropertySchema(BaseModel):
    type: str
    description: Optional[str] = None
    enum: Optional[list[str]] = None


class OpenAIFunctionParametersSchema(BaseModel):
    type: str = "object"
    properties: dict[str, OpenAIFunctionPropertySchema] = Field(default_factory=dict)
    required: list[str] = Field(default_factory=list)


class OpenAIFunctionSchema(BaseModel):
    name: str
    description: str = ""
    parameters: OpenAIFunctionParametersSchema = Field(default_factory=OpenAIFunctionParametersSchema)
    strict: bool = False


class OpenAIFunctionToolSchema(BaseModel):
    type: str = "function"
    function: OpenAIFunctionSchema


class OpenAIFunctionParsedSchema(BaseModel):
    name: str
    arguments: str  # JSON string


class OpenAIFunctionCallSchema(BaseModel):
    name: str
    arguments: dict[str, Any]

    @staticmethod
    def from_openai_function_parsed_schema(parsed: OpenAIFunctionParsedSchema) -> tuple["OpenAIFunctionCallSchema", bool]:
        """Returns (call, has_decode_error)."""
        err = False
        try:
            args = json.loads(parsed.arguments)
        except json.JSONDecodeError:
            args, err = {}, True
        if not isinstance(args, dict):
            args, err = {}, True
        return OpenAIFunctionCallSchema(name=parsed.name, arguments=args), err


class OpenAIFunctionToolCall(BaseModel):
    id: str
    type: Literal["function"] = "function"
    function: OpenAIFunctionCallSchema


class ToolResponse(BaseModel):
    text: Optional[str] = None
    image: Optional[list[Any]] = None
    video: Optional[list[Any]] = None

    def is_empty(self) -> bool:
        return not self.text and not self.image and not self.video

    def is_text_only(self) -> bool:
        return bool(self.text) and not self.image and not self.video
