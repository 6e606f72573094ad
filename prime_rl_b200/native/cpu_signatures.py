"""ctypes signatures of ``libprb200_cpu.so`` (``csrc/cpu/cpu_optim.cpp``)."""

from ctypes import c_float, c_int, c_longlong, c_void_p

P, I, L, F = c_void_p, c_int, c_longlong, c_float

CPU_SIGNATURES = {
    "prb_cpu_adamw_step": [P, P, P, P, I, P, I, L, I, F, F, F, F, F, F],
    "prb_cpu_sign_sgd_step": [P, P, I, P, I, L, F, F, F],
    "prb_cpu_bf16_to_fp32": [P, P, L, I],
}
