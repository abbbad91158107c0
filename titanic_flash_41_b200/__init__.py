"""tflash: a B200-native (sm_100a) tensor/expert-parallel inference engine and
OpenAI-compatible server.  Package map:

config      typed model / engine / server configuration
formats     number formats, checkpoint scan, shard plan, staged atlas, KV page rows
models      PyTorch oracle of the model, CUDA engine, draft head, vision tower, Engram
ops         ctypes bindings of the sm_100a kernels and their CPU oracles
parallel    process bootstrap, collectives, symmetric memory, control plane
spec        counter RNG, samplers, block verification, proposal policies
serve       worker loop, scheduler, session cache, snapshots, host/disk tiers
api         HTTP server, protocol normaliser, chat template, tool-call parser, context transport
utils       tracing, event log, build helpers
"""
__version__ = "0.1.0"
