// Kernels around gated mixers and side inputs on float activations and weights.
#include "gate_kernels.cuh"
#define ELEM float
#define FN(name) sllm_##name##_f32
#include "gate_launchers.inc"
