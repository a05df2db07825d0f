// Kernels around gated mixers and side inputs on bfloat16 activations and weights (float norms, gates and sums).
#include "gate_kernels.cuh"
#define ELEM bf16
#define FN(name) sllm_##name##_bf16
#include "gate_launchers.inc"
