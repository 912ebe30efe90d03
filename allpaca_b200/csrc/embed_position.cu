// Embedding with an additive sinusoidal position vector and an RMS norm, in one pass:
//
//   v[2i]   = table[token][2i]   * scale + sin(pos * inv_freq[i])
//   v[2i+1] = table[token][2i+1] * scale + cos(pos * inv_freq[i])
//   x = v / sqrt(mean(v^2) + eps) * w          (norm only when w is given)
//
// into the 32-bit residual stream.  Angles are 32-bit products of the position and a
// frequency the host computed in 64-bit and rounded once; sincosf is the accurate routine.
// One block per row, the row kept in shared memory between the two passes.
#include "common.cuh"

template <typename TW, typename TN>
__global__ void __launch_bounds__(256)
embed_sinusoid_norm_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                           const TW* __restrict__ table, const float* __restrict__ inv_freq,
                           const TN* __restrict__ norm_w, float eps, float scale, float* __restrict__ x,
                           int H, int V) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float red[32];
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    const float pos = (float)positions[t];
    const TW* src = table + (size_t)tok * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = ap_to_float(src[i]) * scale;
        if (inv_freq != nullptr) {
            float sn, cs;
            sincosf(pos * inv_freq[i >> 1], &sn, &cs);
            v += (i & 1) ? cs : sn;
        }
        row_buf[i] = v;
        ss = fmaf(v, v, ss);
    }
    float inv = 1.f;
    if (norm_w != nullptr) {
        ss = ap_block_sum(ss, red);
        inv = 1.0f / sqrtf(ss / (float)H + eps);
    } else {
        __syncthreads();
    }
    float* dst = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        dst[i] = norm_w != nullptr ? row_buf[i] * inv * ap_to_float(norm_w[i]) : row_buf[i];
}

// inv_freq: [H/2] 32-bit or null (no position vector); norm_w: [H] in norm_dtype or null (no norm).
AP_EXPORT int ap_embed_sinusoid_norm(const int* tokens, const int* positions, const void* table, int table_dtype,
                                     const float* inv_freq, const void* norm_w, int norm_dtype, float eps, float scale,
                                     float* x, int T, int H, int V, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && V > 0, "embed_sinusoid_norm: bad sizes T=%d H=%d V=%d", T, H, V);
    AP_REQUIRE(inv_freq == nullptr || H % 2 == 0, "embed_sinusoid_norm: sine and cosine alternate, the width %d is odd", H);
    AP_REQUIRE((size_t)H * 4 <= 200 * 1024, "embed_sinusoid_norm: width %d does not fit the row buffer", H);
    if (T == 0) return AP_OK;
    const size_t smem = (size_t)H * sizeof(float);
    // The first kernel of a step is launched in plain stream order (see ap_embed_gather).
#define LAUNCH(TW, TN)                                                                                       \
    do {                                                                                                     \
        auto kern = embed_sinusoid_norm_kernel<TW, TN>;                                                      \
        if (smem > 48 * 1024) {                                                                              \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            AP_REQUIRE(e == cudaSuccess, "embed_sinusoid_norm: cannot reserve %zu bytes of shared memory", smem); \
        }                                                                                                    \
        kern<<<T, 256, smem, stream>>>(tokens, positions, (const TW*)table, inv_freq, (const TN*)norm_w, eps, \
                                       scale, x, H, V);                                                      \
    } while (0)
    if (table_dtype == AP_F32 && norm_dtype == AP_F32) LAUNCH(float, float);
    else if (table_dtype == AP_BF16 && norm_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else if (table_dtype == AP_BF16 && norm_dtype == AP_F32) LAUNCH(bf16, float);
    else if (table_dtype == AP_F32 && norm_dtype == AP_BF16) LAUNCH(float, bf16);
    else AP_REQUIRE(false, "embed_sinusoid_norm: unknown dtypes table=%d norm=%d", table_dtype, norm_dtype);
#undef LAUNCH
    AP_CHECK_LAUNCH("embed_sinusoid_norm");
    return AP_OK;
}
