from .agent_loop import AgentLoopBase, AgentLoopManager, AgentLoopMetrics, AgentLoopOutput, AgentLoopWorker, get_agent_loop_class, register
from .single_turn_agent_loop import SingleTurnAgentLoop
from .tool_agent_loop import ToolAgentLoop
from .tool_parser import FunctionCall, ToolParser, get_tool_parser

__all__ = ["AgentLoopBase", "AgentLoopManager", "AgentLoopMetrics", "AgentLoopOutput", "AgentLoopWorker", "SingleTurnAgentLoop",
           "ToolAgentLoop", "FunctionCall", "ToolParser", "get_tool_parser", "get_agent_loop_class", "register"]
