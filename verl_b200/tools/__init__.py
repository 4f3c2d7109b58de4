from .base_tool import BaseTool  # noqa: F401
from .function_tool import FunctionTool, function_to_schema  # noqa: F401
from .registry import initialize_tools_from_config  # noqa: F401
from .schemas import *  # noqa: F401,F403
