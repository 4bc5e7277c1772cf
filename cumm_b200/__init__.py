"""cumm_b200: a B200 (sm_100a) implementation of the sparse-convolution hot path of cumm.

Public surface (names as in the reference):

    cumm_b200.tensorview.gemm   GemmAlgoDesp, ConvAlgoDesp, GemmParams, ConvParams, enums,
                                run_nvrtc_gemm_kernel, run_nvrtc_conv_kernel
    cumm_b200.gemm.main         GemmMainUnitTest  (matmul2, get_all_algo_desp, extract_mnk, ...)
    cumm_b200.conv.main         ConvMainUnitTest  (implicit_gemm2, get_all_conv_algo_desp, ...)

The compute lives in ``libcumm_b200.so`` (hand-written CUDA, C ABI in include/cumm_b200.h).
"""
__version__ = "0.1.0"
