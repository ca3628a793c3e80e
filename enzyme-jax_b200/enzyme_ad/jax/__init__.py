from enzyme_ad.jax.primitives import (  # noqa: F401
    cpp_call,
    ffi_call,
    hlo_call,
    enzyme_jax_ir,
    XLAPipeline,
    JaXPipeline,
    B200Pipeline,
    optimize_module,
    export,
    full_optimization_pass_pipeline,
    optimization_passes,
    vjp,
    register_ffi_targets,
)
from enzyme_ad.jax.hlo_matcher import MatchError, match_llama_forward, rewrite_to_custom_calls  # noqa: F401

