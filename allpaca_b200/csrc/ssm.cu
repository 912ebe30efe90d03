// A selective state-space mixer in its recurrent form (state-space duality, one scalar decay
// per head), with the state a request carries from step to step:
//
//   causal_conv_silu   u_t[c] = silu(b[c] + sum_j w[c][j] * in_{t-(taps-1)+j}[c])     (in_t = 0 for t < 0)
//   conv_state_update  the last taps-1 inputs of every sequence, for its next step
//   ssm_scan           dt = softplus(raw + dt_bias[h]);  S_t = exp(-exp(A_log[h]) dt) S_{t-1} + dt B_t x_t^T;
//                      y_t = S_t^T C_t + D[h] x_t                                        (S: [N, vdim] per head)
//   gated_group_rmsnorm  out = rmsnorm_per_group(y * silu(z)) * w
//
// Everything that enters the recurrence is 32-bit: inputs are read as 32-bit floats, decays,
// step sizes, exponentials and the state itself are 32-bit, and so are the norm's sums.
// A sequence's rows are found through seq_start; its state row through state_slots; a
// portion whose first row has position 0 starts from a zero state.  Nothing is decided
// on the host, so a step of these kernels can be replayed from a CUDA graph.
#include "common.cuh"

__device__ __forceinline__ float ssm_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ssm_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// ---- causal convolution per channel, with SiLU -----------------------------------------
// in: [T, ld_in] 32-bit, the convolved channels start at column `col0`; out: [T, C] 32-bit.
// state: [slots][taps-1][C] 32-bit, the inputs at positions first-(taps-1) .. first-1.
__global__ void causal_conv_silu_kernel(const float* __restrict__ in, long long ld_in, int col0,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        const float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                                        const int* __restrict__ positions, const int* __restrict__ state_slots,
                                        float* __restrict__ out, int T, int C, int taps) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const size_t n = (size_t)T * C;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(e / C), c = (int)(e - (size_t)t * C);
        const int s = token_seq[t];
        const int first_row = seq_start[s];
        const int pos = positions[t];
        const int local = t - first_row;                       // row of the sequence's portion
        const float* st = state + (size_t)state_slots[s] * state_stride;
        float a = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;                     // how many tokens before this one
            float v = 0.f;
            if (pos - back >= 0) {
                if (local - back >= 0) v = in[(size_t)(t - back) * ld_in + col0 + c];
                else v = st[(size_t)(taps - 1 + (local - back)) * C + c];
            }
            a = fmaf(w[(size_t)c * taps + j], v, a);
        }
        out[e] = ssm_silu(a);
    }
}

__global__ void conv_state_update_kernel(const float* __restrict__ in, long long ld_in, int col0,
                                         float* __restrict__ state, long long state_stride,
                                         const int* __restrict__ seq_start, const int* __restrict__ positions,
                                         const int* __restrict__ state_slots, int C, int taps) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const int s = blockIdx.x;
    const int a = seq_start[s], n = seq_start[s + 1] - a;
    if (n <= 0) return;
    const int first_pos = positions[a];
    float* st = state + (size_t)state_slots[s] * state_stride;
    const int keep = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        // slot k holds the input `keep - k` tokens before the next step's first one; ascending k
        // reads old slots only at higher indices than it has written
        for (int k = 0; k < keep; ++k) {
            const int local = n - keep + k;                    // row of this portion, < 0: from before it
            float v;
            if (local >= 0) v = in[(size_t)(a + local) * ld_in + col0 + c];
            else if (first_pos + local >= 0) v = st[(size_t)(keep + local) * C + c];
            else v = 0.f;
            st[(size_t)k * C + c] = v;
        }
    }
}

AP_EXPORT int ap_causal_conv_silu(const float* in, long long ld_in, int col0, const float* w, const float* bias,
                                  float* state, long long state_stride, const int* token_seq, const int* seq_start,
                                  const int* positions, const int* state_slots, float* out, int T, int nseq, int C,
                                  int taps, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nseq >= 0 && C > 0 && taps >= 1 && ld_in >= col0 + C, "causal_conv_silu: bad sizes");
    AP_REQUIRE(taps == 1 || state != nullptr, "causal_conv_silu: a convolution over several tokens needs its state");
    if (T == 0) return AP_OK;
    long long blocks = ((long long)T * C + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    AP_CHECK_PDL_LAUNCH("causal_conv_silu",
                        ap_launch_pdl(causal_conv_silu_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, in, ld_in,
                                      col0, w, bias, (const float*)state, state_stride, token_seq, seq_start, positions,
                                      state_slots, out, T, C, taps));
    if (taps > 1 && nseq > 0) {
        const dim3 grid((unsigned)nseq, (unsigned)((C + 255) / 256));
        AP_CHECK_PDL_LAUNCH("conv_state_update",
                            ap_launch_pdl(conv_state_update_kernel, grid, dim3(256), 0, stream, in, ld_in, col0, state,
                                          state_stride, seq_start, positions, state_slots, C, taps));
    }
    return AP_OK;
}

// ---- the recurrence ---------------------------------------------------------------------
// One CTA per (sequence, head, block of value columns).  A thread holds NPT state entries of one
// value column: the column's N entries are spread over NP neighbouring lanes (NP a power of two
// up to 32), whose partial sums of y meet by shuffles.  Tokens come SCAN_CHUNK at a time through
// two shared-memory buffers filled by asynchronous copies: while one chunk is computed the next
// one is on its way, so the chain over the tokens never waits for memory.
#define NPT 16                   // state entries per thread at most
#define SCAN_CHUNK 16

__device__ __forceinline__ void scan_copy4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_copy16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int PER>               // state entries a thread holds: N <= PER * NP
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const float* __restrict__ xbc, long long ld_xbc,           // [T, inner + 2 G N]: x | B | C
                const float* __restrict__ dt_raw, long long ld_dt,         // [T, .]: column h is head h
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, long long state_stride,         // [slots][heads][N][vdim]
                const int* __restrict__ seq_start, const int* __restrict__ positions,
                const int* __restrict__ state_slots, float* __restrict__ y, // [T, inner]
                int heads, int groups, int N, int vdim, int NP, int cols, int vec) {
    extern __shared__ __align__(16) float sm[];
    ap_pdl_trigger();
    ap_pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y;
    const int a = seq_start[s], n = seq_start[s + 1] - a;
    if (n <= 0) return;
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const int col0 = blockIdx.z * cols;                      // first value column of this CTA
    const int ncols = min(cols, vdim - col0);
    const int vl = threadIdx.x / NP, part = threadIdx.x % NP;
    const int v = col0 + vl;
    const bool live = vl < ncols;
    // one buffer: x [CHUNK][cols], B [CHUNK][N], C [CHUNK][N], dt [CHUNK] (raw, then the step size), decay [CHUNK]
    const int XS = (cols + 3) / 4 * 4, NS = (N + 3) / 4 * 4;
    const int buf_floats = SCAN_CHUNK * (XS + 2 * NS) + 2 * SCAN_CHUNK;
    float* st = state + (size_t)state_slots[s] * state_stride + (size_t)h * N * vdim;
    const bool fresh = positions[a] == 0;
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int nn = part + i * NP;
        S[i] = (!fresh && live && nn < N) ? st[(size_t)nn * vdim + v] : 0.f;
    }
    const float neg_a = -expf(a_log[h]);
    const float bias = dt_bias ? dt_bias[h] : 0.f;
    const float dskip = d_skip ? d_skip[h] : 0.f;

    auto stage = [&](int t0, float* buf) {
        const int cnt = min(SCAN_CHUNK, n - t0);
        float* x_b = buf;
        float* b_b = x_b + SCAN_CHUNK * XS;
        float* c_b = b_b + SCAN_CHUNK * NS;
        float* dt_b = c_b + SCAN_CHUNK * NS;
        if (vec) {
            const int x4 = ncols / 4, n4 = N / 4;
            for (int i = threadIdx.x; i < cnt * x4; i += blockDim.x) {
                const int r = i / x4, d = (i - r * x4) * 4;
                scan_copy16(x_b + r * XS + d, xbc + (size_t)(a + t0 + r) * ld_xbc + (size_t)h * vdim + col0 + d);
            }
            for (int i = threadIdx.x; i < cnt * n4 * 2; i += blockDim.x) {
                const int which = i / (cnt * n4), j = i - which * cnt * n4;
                const int r = j / n4, d = (j - r * n4) * 4;
                scan_copy16((which ? c_b : b_b) + r * NS + d,
                            xbc + (size_t)(a + t0 + r) * ld_xbc + inner + (size_t)(which * groups + g) * N + d);
            }
        } else {
            for (int i = threadIdx.x; i < cnt * ncols; i += blockDim.x) {
                const int r = i / ncols, d = i - r * ncols;
                scan_copy4(x_b + r * XS + d, xbc + (size_t)(a + t0 + r) * ld_xbc + (size_t)h * vdim + col0 + d);
            }
            for (int i = threadIdx.x; i < cnt * N * 2; i += blockDim.x) {
                const int which = i / (cnt * N), j = i - which * cnt * N;
                const int r = j / N, d = j - r * N;
                scan_copy4((which ? c_b : b_b) + r * NS + d,
                           xbc + (size_t)(a + t0 + r) * ld_xbc + inner + (size_t)(which * groups + g) * N + d);
            }
        }
        if (threadIdx.x < cnt) scan_copy4(dt_b + threadIdx.x, dt_raw + (size_t)(a + t0 + threadIdx.x) * ld_dt + h);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    stage(0, sm);
    int which_buf = 0;
    for (int t0 = 0; t0 < n; t0 += SCAN_CHUNK, which_buf ^= 1) {
        const int cnt = min(SCAN_CHUNK, n - t0);
        float* buf = sm + which_buf * buf_floats;
        if (t0 + SCAN_CHUNK < n) {
            stage(t0 + SCAN_CHUNK, sm + (which_buf ^ 1) * buf_floats);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float* x_s = buf;
        float* b_s = x_s + SCAN_CHUNK * XS;
        float* c_s = b_s + SCAN_CHUNK * NS;
        float* dt_s = c_s + SCAN_CHUNK * NS;
        if (threadIdx.x < cnt) {
            const float dtv = ssm_softplus(dt_s[threadIdx.x] + bias);
            dt_s[threadIdx.x] = dtv;
            dt_s[SCAN_CHUNK + threadIdx.x] = expf(neg_a * dtv);
        }
        __syncthreads();
        for (int r = 0; r < cnt; ++r) {
            const float dtv = dt_s[r], decay = dt_s[SCAN_CHUNK + r];
            const float xv = live ? x_s[r * XS + vl] : 0.f;
            const float dx = dtv * xv;
            float acc = 0.f;
            const float* br = b_s + r * NS + part;
            const float* cr = c_s + r * NS + part;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                if (part + i * NP < N) {
                    S[i] = fmaf(decay, S[i], dx * br[i * NP]);
                    acc = fmaf(S[i], cr[i * NP], acc);
                }
            }
            for (int o = NP >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && part == 0) y[(size_t)(a + t0 + r) * inner + (size_t)h * vdim + v] = fmaf(dskip, xv, acc);
        }
        __syncthreads();                                     // this buffer is filled again two chunks on
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int nn = part + i * NP;
            if (nn < N) st[(size_t)nn * vdim + v] = S[i];
        }
    }
}

AP_EXPORT int ap_ssm_scan(const float* xbc, long long ld_xbc, const float* dt_raw, long long ld_dt,
                          const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                          long long state_stride, const int* seq_start, const int* positions, const int* state_slots,
                          float* y, int T, int nseq, int heads, int groups, int N, int vdim, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nseq >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && N > 0 && vdim > 0,
               "ssm_scan: bad sizes heads=%d groups=%d state=%d vdim=%d", heads, groups, N, vdim);
    AP_REQUIRE(N <= NPT * 32, "ssm_scan: a state of %d entries per column exceeds %d", N, NPT * 32);
    AP_REQUIRE(state && a_log && state_stride >= (long long)heads * N * vdim, "ssm_scan: the state is missing or too small");
    if (T == 0 || nseq == 0) return AP_OK;
    int NP = 1;
    while (NP * NPT < N) NP *= 2;
    // at least four lanes to a column, so that a head of few columns still fills warps; and more of them
    // (shorter chains per thread, more warps) while the step's columns do not fill the GPU: the loop over
    // a sequence's tokens is a chain of dependent instructions that only other warps can hide
    while (NP < 4 && NP < N) NP *= 2;
    while (NP < 32 && NP < N && (long long)nseq * heads * vdim * NP / 32 < 148 * 16) NP *= 2;
    const int per = (N + NP - 1) / NP;
    // value columns per CTA: CTAs of four warps, many of them, rather than few large ones: the loop over a
    // sequence's tokens is a chain, and what hides its latency is other chains on the same SM
    int cols = 128 / NP;
    if (cols < 1) cols = 1;
    if (cols > vdim) cols = vdim;
    int threads = (cols * NP + 31) / 32 * 32;
    cols = threads / NP;
    if (cols >= 4) cols = cols / 4 * 4;                     // whole 16-byte runs of x per CTA
    const dim3 grid((unsigned)nseq, (unsigned)heads, (unsigned)((vdim + cols - 1) / cols));
    // 16-byte copies where every run starts on a 16-byte boundary
    const int vec = (cols % 4 == 0 && vdim % 4 == 0 && N % 4 == 0 && ld_xbc % 4 == 0 && ((uintptr_t)xbc & 15) == 0 &&
                     (heads * vdim) % 4 == 0) ? 1 : 0;
    const size_t smem = 2 * ((size_t)SCAN_CHUNK * ((cols + 3) / 4 * 4 + 2 * ((N + 3) / 4 * 4)) + 2 * SCAN_CHUNK) * sizeof(float);
    auto kern = per <= 4 ? ssm_scan_kernel<4> : ssm_scan_kernel<NPT>;
    if (smem > 48 * 1024) {
        AP_REQUIRE(smem <= 200 * 1024, "ssm_scan: a state of %d entries does not fit the staging buffers", N);
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        AP_REQUIRE(e == cudaSuccess, "ssm_scan: cannot reserve %zu bytes of shared memory", smem);
    }
    AP_CHECK_PDL_LAUNCH("ssm_scan", ap_launch_pdl(kern, grid, dim3(threads), smem, stream, xbc, ld_xbc, dt_raw,
                                                  ld_dt, dt_bias, a_log, d_skip, state, state_stride, seq_start,
                                                  positions, state_slots, y, heads, groups, N, vdim, NP, cols, vec));
    return AP_OK;
}

// ---- gate, then RMS norm per slice of the row -------------------------------------------
// y: [T, inner] 32-bit; z: [T, ld_z] 32-bit gate (column 0 of the view); one warp per (row, part).
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ z, long long ld_z,
                           const TW* __restrict__ w, float eps, TO* __restrict__ out, int T, int inner, int parts) {
    ap_pdl_trigger();
    ap_pdl_wait();
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long long)T * parts) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(unit / parts), p = (int)(unit % parts);
    const int width = inner / parts;
    const float* yr = y + (size_t)t * inner + (size_t)p * width;
    const float* zr = z + (size_t)t * ld_z + (size_t)p * width;
    float ss = 0.f;
    for (int i = lane; i < width; i += 32) {
        const float v = yr[i] * ssm_silu(zr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = ap_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    TO* o = out + (size_t)t * inner + (size_t)p * width;
    for (int i = lane; i < width; i += 32) {
        const float v = yr[i] * ssm_silu(zr[i]);
        o[i] = ap_from_float<TO>(v * inv * (w ? ap_to_float(w[(size_t)p * width + i]) : 1.0f));
    }
}

AP_EXPORT int ap_gated_group_rmsnorm(const float* y, const float* z, long long ld_z, const void* w, int w_dtype,
                                     float eps, void* out, int out_dtype, int T, int inner, int parts,
                                     cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && inner > 0 && parts > 0 && inner % parts == 0 && ld_z >= inner,
               "gated_group_rmsnorm: bad sizes inner=%d parts=%d", inner, parts);
    if (T == 0) return AP_OK;
    const dim3 grid((unsigned)(((long long)T * parts + 3) / 4));
#define LAUNCH(TW, TO)                                                                                            \
    AP_CHECK_PDL_LAUNCH("gated_group_rmsnorm",                                                                    \
                        ap_launch_pdl(gated_group_rmsnorm_kernel<TW, TO>, grid, dim3(128), 0, stream, y, z, ld_z, \
                                      (const TW*)w, eps, (TO*)out, T, inner, parts))
    if (w_dtype == AP_F32 && out_dtype == AP_F32) LAUNCH(float, float);
    else if (w_dtype == AP_BF16 && out_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else if (w_dtype == AP_F32 && out_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (w_dtype == AP_BF16 && out_dtype == AP_F32) LAUNCH(bf16, float);
    else AP_REQUIRE(false, "gated_group_rmsnorm: unknown dtypes w=%d out=%d", w_dtype, out_dtype);
#undef LAUNCH
    return AP_OK;
}
