// From a step's projections to queries ready for attention and keys and values in their pages, for mixers
// whose norm spans more than a head and whose rotation is given by rates instead of tables.
//
// One block per token.  In float32 throughout, one rounding at the store:
//   * optional RMS norm over the WHOLE q projection (all heads at once) and over the first `k_norm_cols`
//     elements of the whole k projection, each with its own scale;
//   * rotation of `rot_dims` elements of every q head starting at `q_rot_off`, and of every k head starting at
//     `k_rot_off`: angle = float(position) * rate[i], cosine and sine times `amplitude`; `adjacent` pairs
//     element 2i with 2i + 1 of the span, otherwise i with i + rot_dims / 2; a pair (u, v) becomes
//     (u cos - v sin, v cos + u sin);
//   * queries: elements [0, q_split) of every head to q_out [T, H, q_split], the rest to q_out2 at
//     q_out2[(t * H + h) * q2_head_stride + q2_off + (d - q_split)] (a mixer that replaces the first part of its
//     queries by a product of them puts the second part where that product's result will stand);
//   * keys [G, kd] and values [Gv, vd] into the token's page (layout [pages, heads, page_size, size], 16-byte
//     chunks permuted where the page tensor's rule says so).
// A token whose row of the block table is negative is padding: nothing is read or written for it.
#include "common.cuh"

#include <math.h>

namespace {

__device__ __forceinline__ float qp_block_sum(float v, float* red) {
    v = pb_warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarp; ++i) total += red[i];
    __syncthreads();
    return total;
}

struct RotArgs {
    const float* rates;
    int dims, adjacent;
    float amplitude;
};

// element d of a head whose rotated span starts at `off`: its value after norm and rotation
template <typename T>
__device__ __forceinline__ float rotated(const T* head, const float* w_head, float inv, int d, int off, const RotArgs& r, const float* cs) {
    const float own = pb_ld(head + d) * inv * (w_head ? w_head[d] : 1.0f);
    const int rel = d - off;
    if (r.rates == nullptr || rel < 0 || rel >= r.dims) return own;
    const int half = r.dims >> 1;
    int i, partner;
    bool first;
    if (r.adjacent) { i = rel >> 1; first = (rel & 1) == 0; partner = first ? d + 1 : d - 1; }
    else { first = rel < half; i = first ? rel : rel - half; partner = first ? d + half : d - half; }
    const float other = pb_ld(head + partner) * inv * (w_head ? w_head[partner] : 1.0f);
    const float c = cs[2 * i], s = cs[2 * i + 1];          // of this token's angle i, made once per token
    return first ? own * c - other * s : own * c + other * s;
}

template <typename T>
__global__ void qkv_prepare_kernel(const T* __restrict__ q_in, long long ldq, const T* __restrict__ k_in, long long ldk,
                                   const T* __restrict__ v_in, long long ldv, const float* __restrict__ q_w,
                                   const float* __restrict__ k_w, int k_norm_cols, float eps, RotArgs rot, int q_rot_off,
                                   int k_rot_off, const int32_t* __restrict__ positions, const int32_t* __restrict__ table_row,
                                   const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                                   T* __restrict__ q_out, int q_split, T* __restrict__ q_out2, long long q2_head_stride,
                                   long long q2_off, T* __restrict__ k_pages, T* __restrict__ v_pages, int H, int qd, int G,
                                   int kd, int Gv, int vd, int swizzle_k, int swizzle_v, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    extern __shared__ float cs[];                          // cosine and sine of the token's angles, times the amplitude
    const int t = blockIdx.x;
    const int row = table_row[t];
    if (row < 0) return;
    const int p = positions[t];
    if (rot.rates != nullptr) {
        for (int i = threadIdx.x; i < rot.dims / 2; i += blockDim.x) {
            float sn, c;
            sincosf((float)p * rot.rates[i], &sn, &c);
            cs[2 * i] = c * rot.amplitude;
            cs[2 * i + 1] = sn * rot.amplitude;
        }
        __syncthreads();
    }
    const T* q = q_in + (size_t)t * ldq;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H * qd; i += blockDim.x) { const float v = pb_ld(q + i); ss += v * v; }
        inv_q = 1.0f / sqrtf(qp_block_sum(ss, red) / (float)(H * qd) + eps);
    }
    for (int i = threadIdx.x; i < H * qd; i += blockDim.x) {
        const int h = i / qd, d = i - h * qd;
        const float v = rotated(q + (size_t)h * qd, q_w ? q_w + (size_t)h * qd : nullptr, inv_q, d, q_rot_off, rot, cs);
        if (d < q_split) pb_st(q_out + ((size_t)t * H + h) * q_split + d, v);
        else pb_st(q_out2 + ((size_t)t * H + h) * q2_head_stride + q2_off + (d - q_split), v);
    }
    if (k_pages == nullptr) return;
    const int page = block_table[(size_t)row * table_stride + p / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    const int in_page = p % page_size;
    const T* k = k_in + (size_t)t * ldk;
    if (k_w != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < k_norm_cols; i += blockDim.x) { const float v = pb_ld(k + i); ss += v * v; }
        inv_k = 1.0f / sqrtf(qp_block_sum(ss, red) / (float)k_norm_cols + eps);
    }
    for (int i = threadIdx.x; i < G * kd; i += blockDim.x) {
        const int g = i / kd, d = i - g * kd;
        // the norm covers the first k_norm_cols elements of the projection; the span a rotation turns lies wholly
        // inside or wholly outside them (the launcher checks)
        const bool normed = k_w != nullptr && i < k_norm_cols;
        const float v = rotated(k + (size_t)g * kd, normed ? k_w + (size_t)g * kd : nullptr, normed ? inv_k : 1.0f, d, k_rot_off, rot, cs);
        T* dst = k_pages + (((size_t)page * G + g) * page_size + in_page) * kd;
        pb_st(dst + pb_kv_elem_offset(d, in_page, swizzle_k), v);
    }
    if (v_pages == nullptr || v_in == nullptr) return;
    const T* vv = v_in + (size_t)t * ldv;
    for (int i = threadIdx.x; i < Gv * vd; i += blockDim.x) {
        const int g = i / vd, d = i - g * vd;
        T* dst = v_pages + (((size_t)page * Gv + g) * page_size + in_page) * vd;
        dst[pb_kv_elem_offset(d, in_page, swizzle_v)] = vv[i];
    }
}

}  // namespace

PB_API int pb_qkv_prepare(const void* q_in, long long ldq, const void* k_in, long long ldk, const void* v_in, long long ldv,
                          int dtype, const float* q_w, const float* k_w, int k_norm_cols, float eps, const float* rates,
                          int rot_dims, int adjacent, float amplitude, int q_rot_off, int k_rot_off, const int32_t* positions,
                          const int32_t* table_row, const int32_t* block_table, int table_stride, int page_size, int num_pages,
                          void* q_out, int q_split, void* q_out2, long long q2_head_stride, long long q2_off, void* k_pages,
                          void* v_pages, int n_tokens, int H, int qd, int G, int kd, int Gv, int vd, int swizzle_k,
                          int swizzle_v, int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && H > 0 && qd > 0, "qkv_prepare: bad sizes");
    PB_REQUIRE(q_in && q_out && positions && table_row, "qkv_prepare: null pointer");
    PB_REQUIRE(q_split >= 0 && q_split <= qd && (q_split == qd || q_out2 != nullptr), "qkv_prepare: queries split at %d of %d", q_split, qd);
    PB_REQUIRE(rates == nullptr || (rot_dims > 0 && rot_dims % 2 == 0 && q_rot_off >= 0 && q_rot_off + rot_dims <= qd),
               "qkv_prepare: a rotation of %d elements from %d does not fit a head of %d", rot_dims, q_rot_off, qd);
    if (k_pages != nullptr) {
        PB_REQUIRE(k_in && block_table && G > 0 && kd > 0 && page_size > 0 && num_pages > 0 && table_stride > 0,
                   "qkv_prepare: keys need pages, tables and sizes");
        PB_REQUIRE(rates == nullptr || (k_rot_off >= 0 && k_rot_off + rot_dims <= kd), "qkv_prepare: the rotation does not fit a key head");
        PB_REQUIRE(k_w == nullptr || (k_norm_cols > 0 && k_norm_cols <= G * kd), "qkv_prepare: key norm over %d of %d", k_norm_cols, G * kd);
        // a rotated span lies wholly inside or wholly outside the normed columns
        if (k_w != nullptr && rates != nullptr)
            for (int g = 0; g < G; ++g) {
                const int lo = g * kd + k_rot_off, hi = lo + rot_dims;
                PB_REQUIRE(hi <= k_norm_cols || lo >= k_norm_cols, "qkv_prepare: the key norm's edge cuts a rotated span");
            }
        PB_REQUIRE(v_pages == nullptr || (v_in && Gv > 0 && vd > 0), "qkv_prepare: values need sizes");
        PB_REQUIRE(!swizzle_k || kd % 8 == 0, "qkv_prepare: permuted key rows need a size in multiples of 8");
        PB_REQUIRE(!swizzle_v || vd % 8 == 0, "qkv_prepare: permuted value rows need a size in multiples of 8");
    }
    PB_REQUIRE(rot_dims <= 8192, "qkv_prepare: a rotation of %d elements", rot_dims);
    if (n_tokens == 0) return 0;
    int work = H * qd;
    if (k_pages != nullptr && G * kd > work) work = G * kd;
    int threads = 64;
    while (threads < 512 && threads < work) threads <<= 1;
    RotArgs rot{rates, rot_dims, adjacent, amplitude};
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(qkv_prepare_kernel<T>, dim3(n_tokens), dim3(threads), rates ? (size_t)rot_dims * sizeof(float) : 0, stream, (const T*)q_in, ldq, (const T*)k_in, ldk,
                   (const T*)v_in, ldv, q_w, k_w, k_norm_cols, eps, rot, q_rot_off, k_rot_off, positions, table_row, block_table,
                   table_stride, page_size, num_pages, (T*)q_out, q_split, (T*)q_out2, q2_head_stride, q2_off, (T*)k_pages,
                   (T*)v_pages, H, qd, G, kd, Gv, vd, swizzle_k, swizzle_v, status)));
    PB_CHECK_LAUNCH("qkv_prepare");
    return 0;
}
