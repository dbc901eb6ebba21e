"""ktir_cpu_b200 — B200-native execution backend for KTIR kernels.

Public surface mirrors ``ktir_cpu`` (ktir_cpu/__init__.py:23-27):
``KTIRInterpreter`` with ``load`` / ``arg_names`` / ``tensor_input_output_sizes`` /
``execute_function`` / ``get_latency_report``, the latency model's ``HardwareConfig`` /
``ExecutionModel`` / ``LatencyReport``, ``KTIRParserBase`` as the parser seam and ``register`` /
``register_parser`` as the op plug-in seam (ktir_cpu/dialects/registry.py:98-136).
"""
from .interpreter import KTIRInterpreter, Session
from .latency import ExecutionModel, HardwareConfig, LatencyReport
from .parser import KTIRParser, KTIRParserBase
from .registry import register, register_parser
from .trace import Unsupported

__all__ = ["KTIRInterpreter", "ExecutionModel", "HardwareConfig", "LatencyReport", "KTIRParser", "KTIRParserBase",
           "Session", "Unsupported", "register", "register_parser"]
