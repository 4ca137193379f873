"""Running a quantized model: the fused decoder, graphed decode, chat, tensor parallel."""

from llmquant_b200.runtime.chat import ChatSession, load_for_chat
from llmquant_b200.runtime.graph_decode import GraphedDecoder, can_graph, graphed_generate

__all__ = ["ChatSession", "GraphedDecoder", "can_graph", "graphed_generate", "load_for_chat"]
