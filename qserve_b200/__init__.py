"""qserve_b200 -- Blackwell (sm_100a) W4A8KV4 kernel library behind QServe's operator API.

`qserve_b200.backend` mirrors the reference's `qserve_backend` functions over the C ABI of
`libqserve_b200.so` (include/qserve_b200.h); the top-level `qserve_backend` package re-exports them under
the reference's module names.  Importing `qserve_b200.backend` (or `qserve_backend`) loads the shared library and
fails loudly if it has not been built (`python -m qserve_b200.build`); there is no CPU fallback.

Unquantised hybrid decoders (attention layers beside recurrent layers, fp32 residual stream) are served by `qserve_b200.engine.Engine`:
`modelcfg` (config.json parsers by architecture name: Rizurax, Toderax), `hybrid` (model, mixers and feed-forwards over csrc/hybrid*.cu),
`cache` (page pool and state slots),
`engine` (scheduler, step function, sampling, trace replay), `cli` (`python -m qserve_b200.cli generate|trace`, `bin/trace_run`).
"""
__all__ = ["backend", "build", "cache", "cli", "decode", "engine", "hybrid", "modelcfg", "tp"]
__version__ = "0.1.0"
