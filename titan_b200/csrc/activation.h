// Gated activations of the feed-forward products: what the epilogue makes of a (gate, up) pair of sums.
//
//   TB_ACT_SILU           silu(g) * u                                                   silu(z) = z / (1 + exp(-z))
//   TB_ACT_GELU_TANH      gelu(g) * u, gelu(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   TB_ACT_SWISH_CLAMPED  g' = min(g, limit), u' = clamp(u, -limit, limit):  g' sigmoid(1.702 g') (u' + 1)
//
// The kind and its one constant travel with a launch (``act``, ``limit``); kind 0 is what every launcher without
// them runs.  tb_gated is the precise form (expf, tanhf: the CUDA-core kernels and the true 32-bit path);
// tb_gated_fast uses the fast exponential and division, for epilogues whose result is rounded to bfloat16.
#pragma once
#define TB_ACT_SILU 0
#define TB_ACT_GELU_TANH 1
#define TB_ACT_SWISH_CLAMPED 2
#define TB_ACT_KINDS 3

#ifdef __CUDACC__
__device__ __forceinline__ float tb_gated(int act, float limit, float g, float u) {
    if (act == TB_ACT_GELU_TANH) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    if (act == TB_ACT_SWISH_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return g / (1.0f + expf(-g)) * u;
}
__device__ __forceinline__ float tb_gated_fast(int act, float limit, float g, float u) {
    if (act == TB_ACT_GELU_TANH) {
        // 0.5 (1 + tanh(y)) = 1 / (1 + exp(-2 y))
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return __fdividef(g, 1.0f + __expf(-2.0f * inner)) * u;
    }
    if (act == TB_ACT_SWISH_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdividef(g, 1.0f + __expf(-1.702f * g)) * (u + 1.0f);
    }
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}
#endif
