from .reasoning_parser import ReasoningParser
from .tool_call_parser import ToolCallItem, ToolCallParser
