"""B200-native LLM inference engine with the capabilities of BlockWayz/agens-engine.

Layout: ``models`` (configs, fp32 oracle, engine-backed models), ``ops`` (launchers of the sm_100a kernels),
``parallel`` (symmetric memory, fused collectives, tensor-parallel launcher), ``utils`` (quantisation, checkpoint
I/O, memory planner, profiles, timing), ``serve`` (scheduler, sampler, OpenAI-compatible server bindings).
The native sources live under ``csrc/`` and are built in-tree into ``agens_engine_b200/lib``.
"""
__version__ = "0.1.0"
