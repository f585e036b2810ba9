"""Runtime services: CUDA graphs, layer streaming (host and disk), staging, planning, capabilities, inspection."""

from .capabilities import PrecisionCapabilities
from .cuda_graph import CUDAGraphEngine
from .memory_planner import MemoryEstimate, MemoryPlanner
from .neuron_scope import NeuronScope
from .resource_manager import DynamicResourceManager, LiveVRAMMonitor, VRAMBudgetExceededError
from .sandbox import PythonSandbox, SandboxError
from .staging import FP8StagingBuffer, NVFP4StagingBuffer, ParameterStager, StagingBuffer
from .streaming import LayerStreamingEngine, StreamingConfig, enable_layer_streaming
from .vram import AutoOffloader, VRAMProfiler

__all__ = ["PrecisionCapabilities", "CUDAGraphEngine", "MemoryEstimate", "MemoryPlanner", "NeuronScope", "DynamicResourceManager",
           "LiveVRAMMonitor", "VRAMBudgetExceededError", "PythonSandbox", "SandboxError", "FP8StagingBuffer", "NVFP4StagingBuffer",
           "ParameterStager", "StagingBuffer", "LayerStreamingEngine", "StreamingConfig", "enable_layer_streaming", "AutoOffloader",
           "VRAMProfiler"]
