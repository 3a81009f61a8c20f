// A selective state-space mixer with scalar decay per head, between its input and output projections:
//
//   pb_causal_conv_silu     u = silu(conv(xBC) + bias) per channel over the last `taps` tokens; what lies before the
//                           step's first token comes from the sequence's carried inputs
//   pb_conv_state_update    the last taps - 1 inputs of every sequence, carried to its next step
//   pb_ssm_scan             dt = softplus(dt + bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x, token by
//                           token, the state [heads, state, head_dim] float32 per sequence, read at the start and written
//                           at the end of the step
//   pb_gated_group_rmsnorm  y * silu(z), brought to unit root mean square in equal parts, times a scale
//
// Decay, step size, softplus, exponentials, the state and the sums over it are float32 whatever the run's type;
// the projections and the convolution's output are of the run's type.  A sequence's tokens are visited in order,
// one after the other, by the same threads: the result does not depend on how a prompt was cut into steps or on
// what else is in the batch.  All kernels find a step's sequences through device arrays (cumulative lengths,
// state slots), with one block row per sequence the arrays have room for: a row whose length is not positive is
// skipped, so the launches have the same shape whatever the step holds and can be recorded.
#include "common.cuh"

#include <math.h>

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ in, long long ld_in, const float* __restrict__ w,
                                        const float* __restrict__ bias, const T* __restrict__ carried, T* __restrict__ out,
                                        const int32_t* __restrict__ token_seq, const int32_t* __restrict__ positions,
                                        const int32_t* __restrict__ q_start, const int32_t* __restrict__ slots, int n_tokens,
                                        int channels, int taps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= channels) return;
    const int seq = token_seq[t];
    if (seq < 0) return;                                   // a padding row
    const int i = positions[t] - q_start[seq];             // the token's index among its sequence's tokens of this step
    const T* old = carried + (size_t)slots[seq] * (taps - 1) * channels;
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {
        const int idx = i - (taps - 1 - j);                // in-step index of the input under tap j
        const float x = idx >= 0 ? pb_ld(in + (size_t)(t - (taps - 1 - j)) * ld_in + c)
                                 : pb_ld(old + (size_t)(taps - 1 + idx) * channels + c);
        acc = fmaf(w[(size_t)c * taps + j], x, acc);
    }
    pb_st(out + (size_t)t * channels + c, silu_f(acc));
}

// Row s of a sequence's carried inputs holds the input at in-step index s - (taps - 1) of its NEXT step.  One thread
// owns a (sequence, channel): it reads rows above the one it writes, in ascending order, so nothing is lost.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ in, long long ld_in, T* __restrict__ carried,
                                         const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int channels, int taps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= channels) return;
    const int first = cu_q[r], n = cu_q[r + 1] - first;
    if (n <= 0) return;
    T* st = carried + (size_t)slots[r] * (taps - 1) * channels;
    for (int s = 0; s < taps - 1; ++s) {
        const int idx = n - (taps - 1) + s;
        st[(size_t)s * channels + c] = idx >= 0 ? in[(size_t)(first + idx) * ld_in + c] : st[(size_t)(taps - 1 + idx) * channels + c];
    }
}

// ---------------------------------------------------------------------------------------------------------
// The scan.  A block is 128 threads = 16 columns p of a head's state x 8 lanes over the state rows n; lane j of a
// column keeps rows n = j, j + 8, ... in registers (NPL of them).  Per token: one decay and step size per head,
// S[n][p] = decay S[n][p] + (dt x[p]) B[n], y[p] = sum_n S[n][p] C[n] (own rows in ascending order, then the
// 8 lanes by three exchanges) + D x[p].  The next token's inputs are fetched while this one's are used.
#define SCAN_COLS 16
#define SCAN_LANES 8

template <typename T, int NPL>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_LANES)
ssm_scan_kernel(const T* __restrict__ u, const T* __restrict__ dt_in, long long ld_dt, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state,
                float* __restrict__ y, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ slots, int heads, int P,
                int N, int groups) {
    pb_grid_dep_launch();
    const int col_blocks = (P + SCAN_COLS - 1) / SCAN_COLS;
    const int h = blockIdx.x / col_blocks;
    const int p = (blockIdx.x % col_blocks) * SCAN_COLS + threadIdx.x / SCAN_LANES;
    const int j = threadIdx.x % SCAN_LANES;
    const int r = blockIdx.y;
    const float neg_a = -expf(a_log[h]), bias = dt_bias[h], skip = d_skip[h];     // written by no kernel: before the wait
    pb_grid_dep_wait();
    const int first = cu_q[r], n_tok = cu_q[r + 1] - first;
    if (n_tok <= 0) return;
    const bool live = p < P;
    const int inner = heads * P, channels = inner + 2 * groups * N;
    const int g = h / (heads / groups);
    const int pp = live ? p : P - 1;                                              // idle columns follow along and store nothing
    float* S = state + (((size_t)slots[r] * heads + h) * N) * P + pp;
    float s[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) { const int n = j + SCAN_LANES * i; s[i] = n < N ? S[(size_t)n * P] : 0.f; }

    const T* row = u + (size_t)first * channels;
    float x = pb_ld(row + h * P + pp), dt_raw = pb_ld(dt_in + (size_t)first * ld_dt + h);
    float b[NPL], c[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int n = j + SCAN_LANES * i;
        b[i] = n < N ? pb_ld(row + inner + g * N + n) : 0.f;
        c[i] = n < N ? pb_ld(row + inner + groups * N + g * N + n) : 0.f;
    }
    for (int t = 0; t < n_tok; ++t) {
        float x_next = 0.f, dt_next = 0.f, b_next[NPL], c_next[NPL];
        const bool more = t + 1 < n_tok;
        const T* nrow = row + channels;
        if (more) {
            x_next = pb_ld(nrow + h * P + pp);
            dt_next = pb_ld(dt_in + (size_t)(first + t + 1) * ld_dt + h);
        }
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int n = j + SCAN_LANES * i;
            b_next[i] = (more && n < N) ? pb_ld(nrow + inner + g * N + n) : 0.f;
            c_next[i] = (more && n < N) ? pb_ld(nrow + inner + groups * N + g * N + n) : 0.f;
        }
        const float dt = softplus_f(dt_raw + bias);
        const float decay = expf(neg_a * dt), dx = dt * x;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            s[i] = fmaf(decay, s[i], dx * b[i]);
            acc = fmaf(s[i], c[i], acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        if (live && j == 0) y[(size_t)(first + t) * inner + h * P + p] = fmaf(skip, x, acc);
        x = x_next;
        dt_raw = dt_next;
#pragma unroll
        for (int i = 0; i < NPL; ++i) { b[i] = b_next[i]; c[i] = c_next[i]; }
        row = nrow;
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) { const int n = j + SCAN_LANES * i; if (n < N) S[(size_t)n * P] = s[i]; }
    }
}

// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ld_z,
                                           const float* __restrict__ w, T* __restrict__ out, int inner, int parts, float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const int t = blockIdx.x, part = blockIdx.y, width = inner / parts;
    const float* yr = y + (size_t)t * inner + (size_t)part * width;
    const T* zr = z + (size_t)t * ld_z + (size_t)part * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = yr[i] * silu_f(pb_ld(zr + i)); ss += v * v; }
    ss = pb_warp_sum(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarp; ++i) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    T* o = out + (size_t)t * inner + (size_t)part * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        pb_st(o + i, yr[i] * silu_f(pb_ld(zr + i)) * inv * w[(size_t)part * width + i]);
}

template <typename TI, typename TO>
__global__ void scaled_sum_kernel(const TI* __restrict__ a, float sa, const TI* __restrict__ b, float sb, TO* __restrict__ out, long long n) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pb_st(out + i, sa * pb_ld(a + i) + sb * pb_ld(b + i));
}

}  // namespace

// in: the step's [x | B | C] columns of the input projection, [n_tokens, channels] with row stride ld_in; w float32
// [channels, taps] (last column: the current token); carried [slots, taps - 1, channels]; out [n_tokens, channels] dense.
PB_API int pb_causal_conv_silu(const void* in, long long ld_in, const float* w, const float* bias, const void* carried, void* out,
                               int dtype, const int32_t* token_seq, const int32_t* positions, const int32_t* q_start,
                               const int32_t* slots, int n_tokens, int channels, int taps, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && channels > 0 && taps >= 1 && ld_in >= channels, "causal_conv_silu: bad sizes");
    PB_REQUIRE(in && w && bias && out && token_seq && positions && q_start && slots && (taps == 1 || carried), "causal_conv_silu: null pointer");
    if (n_tokens == 0) return 0;
    PB_REQUIRE((channels + 127) / 128 < 65536, "causal_conv_silu: %d channels in one launch", channels);
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(causal_conv_silu_kernel<T>, dim3(n_tokens, (channels + 127) / 128), dim3(128), 0, stream, (const T*)in, ld_in, w, bias,
                   (const T*)carried, (T*)out, token_seq, positions, q_start, slots, n_tokens, channels, taps)));
    PB_CHECK_LAUNCH("causal_conv_silu");
    return 0;
}

// cu_q [n_seqs + 1], slots [n_seqs]: a sequence whose length cu_q[r + 1] - cu_q[r] is not positive is skipped.
PB_API int pb_conv_state_update(const void* in, long long ld_in, void* carried, int dtype, const int32_t* cu_q, const int32_t* slots,
                                int n_seqs, int channels, int taps, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && channels > 0 && taps >= 1 && ld_in >= channels, "conv_state_update: bad sizes");
    if (n_seqs == 0 || taps == 1) return 0;
    PB_REQUIRE(in && carried && cu_q && slots, "conv_state_update: null pointer");
    PB_REQUIRE(n_seqs < 65536, "conv_state_update: %d sequences in one launch", n_seqs);
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(conv_state_update_kernel<T>, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, stream, (const T*)in, ld_in,
                   (T*)carried, cu_q, slots, channels, taps)));
    PB_CHECK_LAUNCH("conv_state_update");
    return 0;
}

// u: the convolution's output [n_tokens, heads * P + 2 * groups * N] dense, laid out [x | B | C]; dt_in: the step-size
// columns of the input projection, row stride ld_dt; state float32 [slots, heads, N, P]; y float32 [n_tokens, heads * P].
PB_API int pb_ssm_scan(const void* u, const void* dt_in, long long ld_dt, int dtype, const float* dt_bias, const float* a_log,
                       const float* d_skip, float* state, float* y, const int32_t* cu_q, const int32_t* slots, int n_seqs,
                       int heads, int P, int N, int groups, cudaStream_t stream) {
    PB_REQUIRE(n_seqs >= 0 && heads > 0 && P > 0 && N > 0 && groups > 0 && heads % groups == 0, "ssm_scan: bad sizes");
    PB_REQUIRE(N <= 32 * SCAN_LANES, "ssm_scan: a state of %d rows (at most %d)", N, 32 * SCAN_LANES);
    PB_REQUIRE(u && dt_in && dt_bias && a_log && d_skip && state && y && cu_q && slots && ld_dt >= heads, "ssm_scan: null pointer");
    if (n_seqs == 0) return 0;
    PB_REQUIRE(n_seqs < 65536, "ssm_scan: %d sequences in one launch", n_seqs);
    const int col_blocks = (P + SCAN_COLS - 1) / SCAN_COLS;
    const dim3 grid(heads * col_blocks, n_seqs), block(SCAN_COLS * SCAN_LANES);
    const int npl = (N + SCAN_LANES - 1) / SCAN_LANES;
#define SCAN_LAUNCH(NPL)                                                                                                    \
    PB_DISPATCH_DTYPE(dtype, T, (pb_launch(ssm_scan_kernel<T, NPL>, grid, block, 0, stream, (const T*)u, (const T*)dt_in, ld_dt, \
                                           dt_bias, a_log, d_skip, state, y, cu_q, slots, heads, P, N, groups)))
    if (npl <= 4) SCAN_LAUNCH(4);
    else if (npl <= 8) SCAN_LAUNCH(8);
    else if (npl <= 16) SCAN_LAUNCH(16);
    else SCAN_LAUNCH(32);
#undef SCAN_LAUNCH
    PB_CHECK_LAUNCH("ssm_scan");
    return 0;
}

// y float32 [n_tokens, inner]; z: the gate columns of the input projection, row stride ld_z; w float32 [inner];
// out [n_tokens, inner] dense.
PB_API int pb_gated_group_rmsnorm(const float* y, const void* z, long long ld_z, const float* w, void* out, int dtype, int n_tokens,
                                  int inner, int parts, float eps, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inner > 0 && parts > 0 && inner % parts == 0 && ld_z >= inner, "gated_group_rmsnorm: bad sizes");
    PB_REQUIRE(y && z && w && out, "gated_group_rmsnorm: null pointer");
    if (n_tokens == 0) return 0;
    PB_REQUIRE(parts < 65536, "gated_group_rmsnorm: %d parts", parts);
    int threads = 32;
    while (threads < 256 && threads < inner / parts) threads <<= 1;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(gated_group_rmsnorm_kernel<T>, dim3(n_tokens, parts), dim3(threads), 0, stream, y, (const T*)z, ld_z, w, (T*)out, inner,
                   parts, eps)));
    PB_CHECK_LAUNCH("gated_group_rmsnorm");
    return 0;
}

// out = sa * a + sb * b, element by element in float32; a and b of type in_dtype, out of out_dtype.
PB_API int pb_scaled_sum(const void* a, float sa, const void* b, float sb, void* out, int in_dtype, int out_dtype, long long n,
                         cudaStream_t stream) {
    PB_REQUIRE(n >= 0 && a && b && out, "scaled_sum: bad arguments");
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == PB_F32 && out_dtype == PB_F32)
        pb_launch(scaled_sum_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb, (float*)out, n);
    else if (in_dtype == PB_F32 && out_dtype == PB_BF16)
        pb_launch(scaled_sum_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)a, sa, (const float*)b, sb,
                  (__nv_bfloat16*)out, n);
    else if (in_dtype == PB_BF16 && out_dtype == PB_BF16)
        pb_launch(scaled_sum_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, sa,
                  (const __nv_bfloat16*)b, sb, (__nv_bfloat16*)out, n);
    else
        return pb_fail("scaled_sum: unsupported types in=%d out=%d", in_dtype, out_dtype);
    PB_CHECK_LAUNCH("scaled_sum");
    return 0;
}
