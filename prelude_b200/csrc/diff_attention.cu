// Differential attention over paged keys and values, plain form.
//
// A query head holds two score maps.  Map c (0 or 1) of query head h scores the query q[t, h, c, :] against the
// keys of key head 2 g + c, g = h / (heads / kv heads), and both maps weigh the same values, those of value
// head g:
//     S_c[j] = tau(p) * scale * <q_c, k_c[j]>,  j <= p (and j > p - window),   A_c = softmax(S_c) V
//     o = A_0 - lambda * A_1 ;  o <- o / sqrt(mean(o^2) + eps) * out_scale ;  o <- o * sigmoid(gate)   (where a gate is given)
// tau(p) = 1 + coef * ln(floor((p + 1) / every) + 1) is the query temperature (coef 0: none); it multiplies the
// score in float32 instead of the query, which is the same product with one rounding less.
//
// The cache keeps keys as [pages, 2 * kv heads, page_size, dim] (the two maps of a key/value head are two key
// heads, one after the other) and values as [pages, kv heads, page_size, vdim]: dim and vdim are independent.
// pb_kv_write_pages puts a step's keys and values there; it serves any mixer whose keys and values differ in
// head count or size.
//
// This file holds the kernel of the 32-bit path, which is also the fallback of the bfloat16 path and the oracle of
// the tensor-core kernels: one warp per (token, head), float32 arithmetic throughout, keys visited in blocks of
// 32 aligned to absolute positions in ascending order, so that the order of every floating-point operation
// depends on the query's position alone.
#include "common.cuh"

#include <math.h>

#define DA_MAX_D 256
#define DA_MAX_DV 256
#define DA_WARPS 4

template <typename T>
__global__ void kv_write_pages_kernel(const T* __restrict__ k, long long k_stride, const T* __restrict__ v, long long v_stride,
                                      T* __restrict__ k_pages, T* __restrict__ v_pages, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ token_row, const int32_t* __restrict__ block_table,
                                      int table_stride, int page_size, int num_pages, int n_k_heads, int dk, int n_v_heads,
                                      int dv, int k_swizzle, int v_swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int t = blockIdx.x;
    const int row = token_row[t];
    if (row < 0) return;                                   // a padding row of a captured step
    const int pos = positions[t];
    const int page = block_table[(size_t)row * table_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && status) atomicExch(status, 2);
        return;
    }
    const int in_page = pos % page_size;
    const T* kr = k + (size_t)t * k_stride;
    const T* vr = v + (size_t)t * v_stride;
    for (int i = threadIdx.x; i < n_k_heads * dk; i += blockDim.x) {
        const int h = i / dk, d = i % dk;
        k_pages[(((size_t)page * n_k_heads + h) * page_size + in_page) * dk + pb_kv_elem_offset(d, in_page, k_swizzle)] = kr[i];
    }
    for (int i = threadIdx.x; i < n_v_heads * dv; i += blockDim.x) {
        const int h = i / dv, d = i % dv;
        v_pages[(((size_t)page * n_v_heads + h) * page_size + in_page) * dv + pb_kv_elem_offset(d, in_page, v_swizzle)] = vr[i];
    }
}

// k [T, n_k_heads * dk] and v [T, n_v_heads * dv] with row strides in elements (columns of a merged projection);
// pages as described above; token_row[t] is the row of block_table of token t's request (-1: no such token).
PB_API int pb_kv_write_pages(const void* k, long long k_stride, const void* v, long long v_stride, void* k_pages, void* v_pages,
                             int dtype, const int32_t* positions, const int32_t* token_row, const int32_t* block_table,
                             int table_stride, int page_size, int num_pages, int n_tokens, int n_k_heads, int dk,
                             int n_v_heads, int dv, int k_swizzle, int v_swizzle, int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_k_heads > 0 && dk > 0 && n_v_heads > 0 && dv > 0, "kv_write_pages: bad sizes");
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "kv_write_pages: bad cache geometry");
    PB_REQUIRE(k && v && k_pages && v_pages && positions && token_row && block_table, "kv_write_pages: null pointer");
    PB_REQUIRE(k_stride >= (long long)n_k_heads * dk && v_stride >= (long long)n_v_heads * dv, "kv_write_pages: a row stride is shorter than its row");
    PB_REQUIRE((!k_swizzle || dk % 8 == 0) && (!v_swizzle || dv % 8 == 0), "kv_write_pages: permuted pages need head sizes in multiples of 8");
    if (n_tokens == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(kv_write_pages_kernel<T>, dim3(n_tokens), dim3(128), 0, stream, (const T*)k, k_stride, (const T*)v, v_stride,
                   (T*)k_pages, (T*)v_pages, positions, token_row, block_table, table_stride, page_size, num_pages,
                   n_k_heads, dk, n_v_heads, dv, k_swizzle, v_swizzle, status)));
    PB_CHECK_LAUNCH("kv_write_pages");
    return 0;
}

__host__ __device__ __forceinline__ float pb_query_temperature(int pos, float coef, int every) {
    return coef == 0.f ? 1.0f : 1.0f + coef * logf((float)((pos + 1) / every + 1));
}

template <typename T>
__global__ void diff_attention_warp_kernel(
    const T* __restrict__ q, long long q_stride, const T* __restrict__ gate, long long gate_stride,
    const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ out,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_row, const int32_t* __restrict__ block_table,
    int table_stride, int page_size, int num_pages, int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim,
    float scale, float temp_coef, int temp_every, float lambda, float norm_eps, float out_scale, int window,
    int k_swizzle, int v_swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float q_s[DA_WARPS][2][DA_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * DA_WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int row = token_row[t];
    if (row < 0) return;
    const int g = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int32_t* table = block_table + (size_t)row * table_stride;
    const float sc = scale * pb_query_temperature(pos, temp_coef, temp_every);

    const T* qrow = q + (size_t)t * q_stride + (size_t)h * 2 * dim;
    for (int i = lane; i < 2 * dim; i += 32) q_s[warp][i / dim][i % dim] = pb_ld(qrow + i);
    __syncwarp();

    float o[2][DA_MAX_DV / 32];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < DA_MAX_DV / 32; ++i) o[c][i] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    bool bad = false;
    const int n_k_heads = 2 * n_kv_heads;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j >= lo && j <= pos;
        float s[2] = {-INFINITY, -INFINITY};
        int page = -1;
        const int in_page = j % page_size;
        if (valid) {
            page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad = true;
                page = -1;
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const T* kr = k_pages + (((size_t)page * n_k_heads + 2 * g + c) * page_size + in_page) * dim;
                    float acc = 0.f;
                    for (int d = 0; d < dim; ++d) acc = fmaf(q_s[warp][c][d], pb_ld(kr + pb_kv_elem_offset(d, in_page, k_swizzle)), acc);
                    s[c] = acc * sc;
                }
            }
        }
        float p[2], corr[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const float m_new = fmaxf(m[c], pb_warp_max(s[c]));
            if (m_new == -INFINITY) { p[c] = 0.f; corr[c] = 1.f; continue; }   // only when every page id of the block was bad
            p[c] = page >= 0 ? expf(s[c] - m_new) : 0.f;
            corr[c] = (m[c] == -INFINITY) ? 0.f : expf(m[c] - m_new);
            l[c] = l[c] * corr[c] + pb_warp_sum(p[c]);
            m[c] = m_new;
#pragma unroll
            for (int i = 0; i < DA_MAX_DV / 32; ++i) o[c][i] *= corr[c];
        }
        const int n_in_block = min(32, pos - base + 1);
        for (int jj = 0; jj < n_in_block; ++jj) {
            const float p0 = __shfl_sync(0xffffffffu, p[0], jj), p1 = __shfl_sync(0xffffffffu, p[1], jj);
            const int pj = __shfl_sync(0xffffffffu, page, jj);
            if (pj < 0) continue;
            const int vin = (base + jj) % page_size;
            const T* vr = v_pages + (((size_t)pj * n_kv_heads + g) * page_size + vin) * vdim;
#pragma unroll
            for (int i = 0; i < DA_MAX_DV / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < vdim) {
                    const float vv = pb_ld(vr + pb_kv_elem_offset(d, vin, v_swizzle));
                    o[0][i] = fmaf(p0, vv, o[0][i]);
                    o[1][i] = fmaf(p1, vv, o[1][i]);
                }
            }
        }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && status) atomicExch(status, 4);
    // the two maps into one head: difference, unit root mean square, scale, gate
    const float inv0 = l[0] > 0.f ? 1.0f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.0f / l[1] : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < DA_MAX_DV / 32; ++i) {
        const int d = lane + 32 * i;
        o[0][i] = d < vdim ? o[0][i] * inv0 - lambda * (o[1][i] * inv1) : 0.f;
        ss += o[0][i] * o[0][i];
    }
    ss = pb_warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)vdim + norm_eps);
    T* orow = out + ((size_t)t * n_heads + h) * vdim;
    const T* grow = gate ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
#pragma unroll
    for (int i = 0; i < DA_MAX_DV / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) {
            float v = o[0][i] * f;
            if (grow) v *= 1.0f / (1.0f + expf(-pb_ld(grow + d)));
            pb_st(orow + d, v);
        }
    }
}

// q [T, heads * 2 * dim] and gate [T, heads * vdim] (or null) with row strides in elements; out [T, heads, vdim] dense;
// k_pages [pages, 2 * kv heads, page_size, dim], v_pages [pages, kv heads, page_size, vdim]; window <= 0: all keys.
PB_API int pb_diff_attention_ref(const void* q, long long q_stride, const void* gate, long long gate_stride, const void* k_pages,
                                 const void* v_pages, void* out, int dtype, const int32_t* positions, const int32_t* token_row,
                                 const int32_t* block_table, int table_stride, int page_size, int num_pages, int n_tokens,
                                 int n_heads, int n_kv_heads, int dim, int vdim, float scale, float temp_coef, int temp_every,
                                 float lambda, float norm_eps, float out_scale, int window, int k_swizzle, int v_swizzle,
                                 int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
               "diff_attention_ref: %d query heads over %d key/value heads", n_heads, n_kv_heads);
    PB_REQUIRE(dim > 0 && dim <= DA_MAX_D && vdim > 0 && vdim <= DA_MAX_DV, "diff_attention_ref: dim=%d, vdim=%d not in 1..%d", dim, vdim, DA_MAX_D);
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0 && temp_every > 0, "diff_attention_ref: bad cache geometry or temperature step");
    PB_REQUIRE(q && k_pages && v_pages && out && positions && token_row && block_table, "diff_attention_ref: null pointer");
    if (n_tokens == 0) return 0;
    long long items = (long long)n_tokens * n_heads;
    long long blocks = (items + DA_WARPS - 1) / DA_WARPS;
    PB_REQUIRE(blocks < (1ll << 31), "diff_attention_ref: too many rows");
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(diff_attention_warp_kernel<T>, dim3((unsigned)blocks), dim3(DA_WARPS * 32), 0, stream, (const T*)q, q_stride,
                   (const T*)gate, gate_stride, (const T*)k_pages, (const T*)v_pages, (T*)out, positions, token_row, block_table,
                   table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, dim, vdim, scale, temp_coef, temp_every,
                   lambda, norm_eps, out_scale, window, k_swizzle, v_swizzle, status)));
    PB_CHECK_LAUNCH("diff_attention_ref");
    return 0;
}
