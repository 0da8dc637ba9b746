from .gemm import grouped_gemm_dgrad, grouped_gemm_fwd, grouped_gemm_wgrad, pad_group_offsets  # noqa: F401
