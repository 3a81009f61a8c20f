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

__device__ __forceinline__ void qp_ld_vec(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void qp_ld_vec(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void qp_st_vec(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void qp_st_vec(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
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


// The same with the token's projections staged in shared memory as float32: one pass over global memory with 16-byte
// loads, sums and rotation partners from shared memory, 16-byte stores.  Takes rows whose q, k and v parts start on
// 16-byte boundaries and have sizes in multiples of 8 (bfloat16) or 4 (float32) elements, heads and split points likewise.
template <typename T>
__global__ void qkv_prepare_staged_kernel(const T* __restrict__ q_in, long long ldq, const T* __restrict__ k_in, long long ldk,
                                          const T* __restrict__ v_in, long long ldv, const float* __restrict__ q_w,
                                          const float* __restrict__ k_w, int k_norm_cols, float eps, RotArgs rot, int q_rot_off,
                                          int k_rot_off, const int32_t* __restrict__ positions, const int32_t* __restrict__ table_row,
                                          const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
                                          T* __restrict__ q_out, int q_split, T* __restrict__ q_out2, long long q2_head_stride,
                                          long long q2_off, T* __restrict__ k_pages, T* __restrict__ v_pages, int H, int qd, int G,
                                          int kd, int Gv, int vd, int swizzle_k, int swizzle_v, int* __restrict__ status) {
    constexpr int VN = 16 / sizeof(T);
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    extern __shared__ float sm[];
    const int nq = H * qd, nk = k_pages ? G * kd : 0;
    float* cs = sm;                                       // cosine and sine of the token's angles
    float* qs = sm + rot.dims;
    float* ks = qs + nq;
    const int t = blockIdx.x;
    const int row = table_row[t];
    if (row < 0) return;
    const int p = positions[t];
    if (rot.rates != nullptr)
        for (int i = threadIdx.x; i < rot.dims / 2; i += blockDim.x) {
            float sn, c;
            sincosf((float)p * rot.rates[i], &sn, &c);
            cs[2 * i] = c * rot.amplitude;
            cs[2 * i + 1] = sn * rot.amplitude;
        }
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x * VN; i < nq; i += blockDim.x * VN) {
        float v[VN];
        qp_ld_vec(q_in + (size_t)t * ldq + i, v);
#pragma unroll
        for (int e = 0; e < VN; ++e) { qs[i + e] = v[e]; ssq += v[e] * v[e]; }
    }
    for (int i = threadIdx.x * VN; i < nk; i += blockDim.x * VN) {
        float v[VN];
        qp_ld_vec(k_in + (size_t)t * ldk + i, v);
#pragma unroll
        for (int e = 0; e < VN; ++e) { ks[i + e] = v[e]; if (i + e < k_norm_cols) ssk += v[e] * v[e]; }
    }
    const float tq = qp_block_sum(ssq, red), tk = qp_block_sum(ssk, red);          // the barriers also publish the staged rows
    const float inv_q = q_w ? 1.0f / sqrtf(tq / (float)nq + eps) : 1.0f;
    const float inv_k = k_w ? 1.0f / sqrtf(tk / (float)k_norm_cols + eps) : 1.0f;
    for (int i = threadIdx.x * VN; i < nq; i += blockDim.x * VN) {
        const int h = i / qd, d0 = i - h * qd;
        float v[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) v[e] = rotated(qs + (size_t)h * qd, q_w ? q_w + (size_t)h * qd : nullptr, inv_q, d0 + e, q_rot_off, rot, cs);
        if (d0 < q_split) qp_st_vec(q_out + ((size_t)t * H + h) * q_split + d0, v);
        else qp_st_vec(q_out2 + ((size_t)t * H + h) * q2_head_stride + q2_off + (d0 - q_split), v);
    }
    if (k_pages == nullptr) return;
    const int page = block_table[(size_t)row * table_stride + p / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    const int in_page = p % page_size;
    for (int i = threadIdx.x * VN; i < nk; i += blockDim.x * VN) {
        const int g = i / kd, d0 = i - g * kd;
        const bool normed = k_w != nullptr && i < k_norm_cols;
        float v[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) v[e] = rotated(ks + (size_t)g * kd, normed ? k_w + (size_t)g * kd : nullptr, normed ? inv_k : 1.0f, d0 + e, k_rot_off, rot, cs);
        T* dst = k_pages + (((size_t)page * G + g) * page_size + in_page) * kd;
        qp_st_vec(dst + pb_kv_elem_offset(d0, in_page, swizzle_k), v);
    }
    if (v_pages == nullptr || v_in == nullptr) return;
    for (int i = threadIdx.x * VN; i < Gv * vd; i += blockDim.x * VN) {
        const int g = i / vd, d0 = i - g * vd;
        T* dst = v_pages + (((size_t)page * Gv + g) * page_size + in_page) * vd;
        *reinterpret_cast<uint4*>(dst + pb_kv_elem_offset(d0, in_page, swizzle_v)) = *reinterpret_cast<const uint4*>(v_in + (size_t)t * ldv + i);
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
    RotArgs rot{rates, rates ? rot_dims : 0, adjacent, amplitude};
    const int vn = dtype == PB_BF16 ? 8 : 4;
    const size_t staged_bytes = ((size_t)rot.dims + (size_t)H * qd + (k_pages ? (size_t)G * kd : 0)) * sizeof(float);
    bool staged = staged_bytes <= 40 * 1024 && qd % vn == 0 && q_split % vn == 0 && ldq % vn == 0 && pb_aligned(q_in, 16) && pb_aligned(q_out, 16) &&
                  (q_split == qd || (q2_head_stride % vn == 0 && q2_off % vn == 0 && pb_aligned(q_out2, 16)));
    if (staged && k_pages != nullptr)
        staged = kd % vn == 0 && ldk % vn == 0 && pb_aligned(k_in, 16) && pb_aligned(k_pages, 16) && k_norm_cols % vn == 0 &&
                 (v_pages == nullptr || (vd % vn == 0 && ldv % vn == 0 && pb_aligned(v_in, 16) && pb_aligned(v_pages, 16)));
    if (staged) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(qkv_prepare_staged_kernel<T>, dim3(n_tokens), dim3(threads >= 128 ? threads / 2 : threads), staged_bytes, stream, (const T*)q_in, ldq,
                       (const T*)k_in, ldk, (const T*)v_in, ldv, q_w, k_w, k_norm_cols, eps, rot, q_rot_off, k_rot_off, positions, table_row,
                       block_table, table_stride, page_size, num_pages, (T*)q_out, q_split, (T*)q_out2, q2_head_stride, q2_off, (T*)k_pages,
                       (T*)v_pages, H, qd, G, kd, Gv, vd, swizzle_k, swizzle_v, status)));
        PB_CHECK_LAUNCH("qkv_prepare");
        return 0;
    }
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(qkv_prepare_kernel<T>, dim3(n_tokens), dim3(threads), rates ? (size_t)rot_dims * sizeof(float) : 0, stream, (const T*)q_in, ldq, (const T*)k_in, ldk,
                   (const T*)v_in, ldv, q_w, k_w, k_norm_cols, eps, rot, q_rot_off, k_rot_off, positions, table_row, block_table,
                   table_stride, page_size, num_pages, (T*)q_out, q_split, (T*)q_out2, q2_head_stride, q2_off, (T*)k_pages,
                   (T*)v_pages, H, qd, G, kd, Gv, vd, swizzle_k, swizzle_v, status)));
    PB_CHECK_LAUNCH("qkv_prepare");
    return 0;
}
