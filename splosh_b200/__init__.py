"""SploshCUDA: the B200 (sm_100a) packed ragged step of Splosh behind a C ABI.

The product is `libsploshcuda.so` (see include/splosh_cuda.h). This package is the thin Python
host over it that mirrors the reference's Swift `Engine` interface
(Sources/SploshRuntime/Engine.swift) for tests and benchmarks. There is no CPU fallback.
"""
from .engine import (Engine, EngineConfig, EngineRow, EngineError, Geometry, Host, StepStats, tiny_geometry, b27_geometry,
                     gemm_q4, gemm_gguf, greedy_accept, library_path, Sampler, Planner, PackSession)

from .draft import DraftModel, DraftConfig, DraftRequest, DraftProposal

__all__ = ["DraftModel", "DraftConfig", "DraftRequest", "DraftProposal", "Engine", "EngineConfig", "EngineRow", "EngineError", "Geometry", "Host", "StepStats", "tiny_geometry",
           "b27_geometry", "gemm_q4", "gemm_gguf", "greedy_accept", "library_path", "Sampler", "Planner", "PackSession"]
