from .agent_loop import AgentLoopBase, AgentLoopManager, AgentLoopOutput, AgentLoopWorker, get_agent_loop_class, register  # noqa: F401
from .single_turn_agent_loop import SingleTurnAgentLoop  # noqa: F401
from .tool_agent_loop import ToolAgentLoop  # noqa: F401
