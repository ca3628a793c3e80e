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
)
