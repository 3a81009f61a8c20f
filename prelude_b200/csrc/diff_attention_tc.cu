// Differential attention on the tensor cores (bfloat16 operands, float32 accumulators and softmax), for prompt
// portions and for decoded tokens.
//
// A block takes a tile of 64 query rows - the tokens of one request's portion times the query heads of one
// key/value head - and walks the request's keys in tiles of 64.  It has eight warps: warps 0..3 hold score map 0 of
// rows 16 w .. 16 w + 15, warps 4..7 score map 1 of the same rows; each is a flash-attention warp with keys of `dim`
// and values of `vdim` (S = Q K^T and O += P V as mma.sync m16n8k16, running maximum and sum in float32, base 2).
// Both maps read the same value tile from shared memory.  The query temperature and the scale multiply the scores in
// float32.  The softmax weights enter the second product as a sum of two bfloat16 numbers (the weight rounded, and
// what the rounding lost), so that the difference of two nearly equal maps does not inherit a bfloat16 rounding of
// its weights.  At the end the warps of map 1 hand their normalised rows over through shared memory and the warps of
// map 0 do the head's epilogue: difference, unit root mean square, scale, gate, store.
//
// Keys and values come from the pages with 16-byte asynchronous copies into padded rows (a permuted page is
// straightened on the way), two tiles in flight where shared memory allows.  A row of keys beyond the request's last
// position, or of a page that a window has given back, is filled with zeros, so that no weight of zero meets a
// value that is not a number.
//
// Decoded tokens have a tile of their own (`tile_seq` null: tile i is token i).  Their keys can be cut into
// `n_splits` ranges, one block each; the blocks then leave unnormalised sums with their maxima and the merge kernel
// below adds them up and does the epilogue.
#include "attention_common.cuh"

struct DiffAttnParams {
    const __nv_bfloat16* q; long long q_stride;          // [T, heads * 2 * dim]
    const __nv_bfloat16* gate; long long gate_stride;    // [T, heads * vdim] or null
    const __nv_bfloat16* k_pages;                        // [pages, 2 * kv heads, page_size, dim]
    const __nv_bfloat16* v_pages;                        // [pages, kv heads, page_size, vdim]
    __nv_bfloat16* out;                                  // [T, heads, vdim]
    const int32_t* block_table; const int32_t* positions; const int32_t* token_row;
    const int32_t* cu_q; const int32_t* tile_seq; const int32_t* tile_tok0;
    float* part_o;                                       // [T, heads, 2, n_splits, vdim]
    float* part_ml;                                      // [T, heads, 2, n_splits, 2]
    int n_splits, stages;
    int n_parts;                                         // partial sums per (token, head, map) that the merge kernel adds up
    int split_weights;                                   // the softmax weights enter O += P V as rounded part plus remainder
    int table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, dim, vdim, group, window;
    int k_swizzle, v_swizzle;
    float scale_log2, temp_coef; int temp_every;
    float lambda, norm_eps, out_scale;
    int* status;
};

__device__ __forceinline__ void ldsm_x4_at(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans_at(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float da_temperature(int pos, float coef, int every) {
    return coef == 0.f ? 1.0f : 1.0f + coef * logf((float)((pos + 1) / every + 1));
}

// NV: 16-column steps of the values at most; KS: 16-element steps of the keys (0: read from the parameters).
// DEC: a decoded token's tile, whose rows (the query heads of one key/value head, sixteen at most) fit one warp: the
// four warps of a map then share every 64-key tile, sixteen keys each, and leave four partial sums per key range,
// which the merge kernel takes as four ranges more.  A single warp walking whole tiles is bound by the latency of
// its own instructions (17 cycles between two of them, measured) and four of them by a quarter of it.
template <int NV, int KS, bool DEC>
__global__ void __launch_bounds__(256) diff_attention_mma_kernel(const DiffAttnParams p) {
    constexpr int NT = DEC ? 2 : 8;                         // 8-key score tiles per warp and key tile
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t4 = lane & 3;
    const int map = warp >> 2, row0 = DEC ? 0 : (warp & 3) * 16, key_off = DEC ? (warp & 3) * 16 : 0;
    const int g = blockIdx.y, split = blockIdx.z;
    const int dim = KS ? KS * 16 : p.dim, vdim = p.vdim, group = p.group;
    const int tpt = 64 / group;
    int tok_first, n_tok;
    if (p.tile_seq) {
        const int seq = p.tile_seq[blockIdx.x], tok0 = p.tile_tok0[blockIdx.x], base = p.cu_q[seq];
        tok_first = base + tok0;
        n_tok = min(tpt, p.cu_q[seq + 1] - base - tok0);
    } else {
        tok_first = blockIdx.x;
        n_tok = 1;
    }
    const int trow = p.token_row[tok_first];
    if (trow < 0) return;                                   // a padding row of a captured step
    const int pos_first = p.positions[tok_first], pos_last = pos_first + n_tok - 1;
    const int lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int kt_lo = lo / 64, kt_hi = pos_last / 64;
    const int per = (kt_hi - kt_lo + p.n_splits) / p.n_splits;
    const int kt_begin = kt_lo + split * per, kt_end = min(kt_hi + 1, kt_begin + per);
    const int32_t* table = p.block_table + (size_t)trow * p.table_stride;

    const int SK = dim + 8, SV = vdim + 8;                  // elements per row in shared memory
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);                 // [2][64][SK]
    const size_t stage_elems = (size_t)2 * 64 * SK + (size_t)64 * SV;
    __nv_bfloat16* stage0 = Qs + (size_t)2 * 64 * SK;                            // per stage: K [2][64][SK], V [64][SV]

    // Four threads share a row of every 64-row tile (queries, keys, values) and take its 16-byte pieces in turn.
    const int lrow = tid >> 2, lsub = tid & 3;
    // queries of both maps: row r is token r / group, head g * group + r % group
    {
        const int tl = lrow / group, hh = lrow % group;
        const bool ok = tl < n_tok;
        const __nv_bfloat16* src = p.q + (size_t)(tok_first + (ok ? tl : 0)) * p.q_stride + (size_t)((g * group + hh) * 2) * dim;
        for (int cc = lsub; cc < 2 * (dim / 8); cc += 4) {
            const int c = cc >= dim / 8 ? 1 : 0, ch = cc - c * (dim / 8);
            cp_async16(Qs + ((size_t)c * 64 + lrow) * SK + ch * 8, src + cc * 8, ok);
        }
    }
    bool bad_page = false;
    auto load_tile = [&](int kt, int st) {
        __nv_bfloat16* Ks = stage0 + (size_t)st * stage_elems;
        __nv_bfloat16* Vs = Ks + (size_t)2 * 64 * SK;
        const int j = kt * 64 + lrow;
        int page = -1;
        if (j >= lo && j <= pos_last) {
            page = table[j / p.page_size];
            if (page >= p.num_pages) { bad_page = true; page = -1; }
        }
        const bool ok = page >= 0;
        const int in_page = j % p.page_size, x = in_page & 7;
        const __nv_bfloat16* k0 = p.k_pages + (((size_t)(ok ? page : 0) * (2 * p.n_kv_heads) + 2 * g) * p.page_size + in_page) * dim;
        const __nv_bfloat16* k1 = k0 + (size_t)p.page_size * dim;
        const __nv_bfloat16* v0 = p.v_pages + (((size_t)(ok ? page : 0) * p.n_kv_heads + g) * p.page_size + in_page) * vdim;
        for (int cc = lsub; cc < dim / 8; cc += 4) {
            const int stored = p.k_swizzle ? (cc ^ x) : cc;
            cp_async16(Ks + (size_t)lrow * SK + cc * 8, k0 + stored * 8, ok);
            cp_async16(Ks + ((size_t)64 + lrow) * SK + cc * 8, k1 + stored * 8, ok);
        }
        for (int cc = lsub; cc < vdim / 8; cc += 4) {
            const int stored = p.v_swizzle ? (cc ^ x) : cc;
            cp_async16(Vs + (size_t)lrow * SV + cc * 8, v0 + stored * 8, ok);
        }
    };

    // this thread's two rows (gid and gid + 8 of the warp's sixteen): position and score factor
    int row_pos[2];
    float sc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = row0 + gid + 8 * h, tl = r / group;
        row_pos[h] = tl < n_tok ? pos_first + tl : -1;
        sc[h] = p.scale_log2 * da_temperature(max(row_pos[h], 0), p.temp_coef, p.temp_every);
    }
    // a warp whose sixteen rows hold no token (a decoded token fills few rows of its tile) copies and waits with the
    // others and computes nothing
    const bool warp_active = DEC || row0 / group < n_tok;
    const bool rows_missing = 64 / group * group < 64 || n_tok < 64 / group;
    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    // per-lane byte offsets of the ldmatrix rows
    const unsigned q_off = (unsigned)(((size_t)map * 64 + row0 + (lane & 15)) * SK + (lane >> 4) * 8) * 2;
    const unsigned k_off = (unsigned)(((size_t)map * 64 + key_off + (lane >> 4) * 8 + (lane & 7)) * SK + ((lane >> 3) & 1) * 8) * 2;
    const unsigned v_off = (unsigned)(((size_t)key_off + ((lane >> 3) & 1) * 8 + (lane & 7)) * SV + (lane >> 4) * 8) * 2;
    const unsigned sQ = smem_u32(Qs);

    if (kt_begin < kt_end) load_tile(kt_begin, 0);
    cp_async_commit();
    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int st = p.stages == 2 ? ((kt - kt_begin) & 1) : 0;
        if (p.stages == 2 && kt + 1 < kt_end) load_tile(kt + 1, st ^ 1);
        cp_async_commit();
        if (p.stages == 2) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        const unsigned sK = smem_u32(stage0 + (size_t)st * stage_elems);
        const unsigned sV = sK + (unsigned)(2 * 64 * SK * 2);
        if (warp_active) {
        // ---- S = Q K^T, 16 rows x 64 keys ----
        float s[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < (KS ? KS : 16); ++kk) {
            if (KS == 0 && kk >= dim / 16) break;
            unsigned qa[4];
            ldsm_x4_at(qa, sQ + q_off + kk * 32);
#pragma unroll
            for (int n2 = 0; n2 < NT / 2; ++n2) {
                unsigned kb[4];
                ldsm_x4_at(kb, sK + k_off + (unsigned)(n2 * 16 * SK * 2) + kk * 32);
                mma_bf16_free(s[2 * n2], qa, kb[0], kb[1]);
                mma_bf16_free(s[2 * n2 + 1], qa, kb[2], kb[3]);
            }
        }
        // ---- scale and temperature, mask (only in tiles that hold a key some row may not see), running maximum ----
        const int j0 = kt * 64;
        const bool edge = rows_missing || j0 + 63 > pos_first || (p.window > 0 && j0 <= pos_last - p.window);
        // four partial maxima (and, below, sums) per row instead of one chain of sixteen
        float pm[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) pm[h][0] = pm[h][1] = pm[h][2] = pm[h][3] = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * sc[e >> 1];
                if (edge) {
                    const int j = j0 + key_off + nt * 8 + 2 * t4 + (e & 1);
                    const int pr = row_pos[e >> 1];
                    v = (j <= pr && (p.window <= 0 || j > pr - p.window)) ? v : -INFINITY;
                }
                s[nt][e] = v;
                pm[e >> 1][(nt & 1) * 2 + (e & 1)] = fmaxf(pm[e >> 1][(nt & 1) * 2 + (e & 1)], v);
            }
        }
        float rmax[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) rmax[h] = fmaxf(fmaxf(pm[h][0], pm[h][1]), fmaxf(pm[h][2], pm[h][3]));
        float mref[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
            const float m_new = fmaxf(m[h], rmax[h]);
            mref[h] = m_new == -INFINITY ? 0.f : m_new;
            if (m_new > m[h]) {                              // the maximum grew: earlier sums shrink
                const float corr = (m[h] == -INFINITY) ? 0.f : ex2_approx(m[h] - m_new);
                m[h] = m_new;
                l[h] *= corr;
#pragma unroll
                for (int i = 0; i < 2 * NV; ++i) { o[i][2 * h] *= corr; o[i][2 * h + 1] *= corr; }
            }
        }
        float ps[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) ps[h][0] = ps[h][1] = ps[h][2] = ps[h][3] = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = ex2_approx(s[nt][e] - mref[e >> 1]);
                s[nt][e] = pv;
                ps[e >> 1][(nt & 1) * 2 + (e & 1)] += pv;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l[h] += (ps[h][0] + ps[h][1]) + (ps[h][2] + ps[h][3]);
        // ---- O += P V, the weights as rounded part plus remainder ----
#pragma unroll
        for (int ks = 0; ks < NT / 2; ++ks) {
            unsigned hi[4], lw[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float x0 = s[2 * ks + (a >> 1)][(a & 1) * 2], x1 = s[2 * ks + (a >> 1)][(a & 1) * 2 + 1];
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(x0, x1);
                const float2 back = __bfloat1622float2(h2);
                hi[a] = *reinterpret_cast<const unsigned*>(&h2);
                lw[a] = pack_bf16(x0 - back.x, x1 - back.y);
            }
#pragma unroll
            for (int d2 = 0; d2 < NV; ++d2) {
                if (d2 * 16 < vdim) {
                    unsigned vb[4];
                    ldsm_x4_trans_at(vb, sV + v_off + (unsigned)(ks * 16 * SV * 2) + d2 * 32);
                    mma_bf16_free(o[2 * d2], hi, vb[0], vb[1]);
                    mma_bf16_free(o[2 * d2 + 1], hi, vb[2], vb[3]);
                    if (p.split_weights) {
                        mma_bf16_free(o[2 * d2], lw, vb[0], vb[1]);
                        mma_bf16_free(o[2 * d2 + 1], lw, vb[2], vb[3]);
                    }
                }
            }
        }
        }
        __syncthreads();
        if (p.stages != 2 && kt + 1 < kt_end) load_tile(kt + 1, 0);
    }
    cp_async_wait<0>();
    if (bad_page && p.status) atomicExch(p.status, 6);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }

    if (DEC || p.n_splits > 1) {
        // unnormalised sums with their maximum and sum, for the merge kernel
        const int n_parts = DEC ? 4 * p.n_splits : p.n_splits, part = DEC ? 4 * split + (warp & 3) : split;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (row_pos[h] < 0) continue;
            const int r = row0 + gid + 8 * h;
            const int tok = tok_first + r / group, head = g * group + r % group;
            const size_t at = ((((size_t)tok * p.n_heads + head) * 2 + map) * n_parts + part);
            if (t4 == 0) { p.part_ml[at * 2] = m[h]; p.part_ml[at * 2 + 1] = l[h]; }
            float* po = p.part_o + at * vdim;
#pragma unroll
            for (int nt = 0; nt < 2 * NV; ++nt)
                if (nt * 8 < vdim) *reinterpret_cast<float2*>(po + nt * 8 + 2 * t4) = make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
        }
        return;
    }

    // ---- the head's epilogue: map 1 hands over, map 0 combines ----
    __syncthreads();                                         // everyone is done with the tiles
    float* A2 = reinterpret_cast<float*>(smem);              // [64][vdim + 4]
    const int SA = vdim + 4;
    const float inv[2] = {l[0] > 0.f ? 1.0f / l[0] : 0.f, l[1] > 0.f ? 1.0f / l[1] : 0.f};
    if (map == 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* dst = A2 + (size_t)(row0 + gid + 8 * h) * SA;
#pragma unroll
            for (int nt = 0; nt < 2 * NV; ++nt)
                if (nt * 8 < vdim) *reinterpret_cast<float2*>(dst + nt * 8 + 2 * t4) = make_float2(o[nt][2 * h] * inv[h], o[nt][2 * h + 1] * inv[h]);
        }
    }
    __syncthreads();
    if (map == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float* src = A2 + (size_t)(row0 + gid + 8 * h) * SA;
            float ss = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2 * NV; ++nt) {
                if (nt * 8 < vdim) {
                    const float2 a2 = *reinterpret_cast<const float2*>(src + nt * 8 + 2 * t4);
                    o[nt][2 * h] = o[nt][2 * h] * inv[h] - p.lambda * a2.x;
                    o[nt][2 * h + 1] = o[nt][2 * h + 1] * inv[h] - p.lambda * a2.y;
                    ss += o[nt][2 * h] * o[nt][2 * h] + o[nt][2 * h + 1] * o[nt][2 * h + 1];
                }
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (row_pos[h] < 0) continue;
            const float f = p.out_scale / sqrtf(ss / (float)vdim + p.norm_eps);
            const int r = row0 + gid + 8 * h;
            const int tok = tok_first + r / group, head = g * group + r % group;
            __nv_bfloat16* dst = p.out + ((size_t)tok * p.n_heads + head) * vdim;
            const __nv_bfloat16* gt = p.gate ? p.gate + (size_t)tok * p.gate_stride + (size_t)head * vdim : nullptr;
#pragma unroll
            for (int nt = 0; nt < 2 * NV; ++nt) {
                if (nt * 8 < vdim) {
                    const int col = nt * 8 + 2 * t4;
                    float v0 = o[nt][2 * h] * f, v1 = o[nt][2 * h + 1] * f;
                    if (gt) {
                        v0 *= 1.0f / (1.0f + expf(-__bfloat162float(gt[col])));
                        v1 *= 1.0f / (1.0f + expf(-__bfloat162float(gt[col + 1])));
                    }
                    *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(v0, v1);
                }
            }
        }
    }
}

// A block of eight warps per (token, head): warps 0..3 on map 0, 4..7 on map 1.  In every warp lane s takes part s's
// maximum and sum (at most 32 parts) and the warp agrees on the common maximum and on each part's share; warp w of a
// map then adds up parts w, w + 4, ... over its columns, all loads issued before the first sum (one round trip to the
// cache instead of one per part), the four warps' sums meet in shared memory, and warp 0 does the head's epilogue.
__global__ void __launch_bounds__(256) diff_attention_merge_kernel(const DiffAttnParams p) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float acc_s[2][4][256];
    const int c = threadIdx.x >> 7, w = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
    const int tok = blockIdx.x / p.n_heads, head = blockIdx.x % p.n_heads;
    if (p.token_row[tok] < 0) return;
    const int vdim = p.vdim, S = p.n_parts;
    const size_t at = ((size_t)tok * p.n_heads + head) * 2 + c;
    float ms = -INFINITY, ls = 0.f;
    if (lane < S) { ms = p.part_ml[(at * S + lane) * 2]; ls = p.part_ml[(at * S + lane) * 2 + 1]; }
    const float* po = p.part_o + at * S * vdim;
    float v[8][8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int part = w + 4 * u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int col = lane + 32 * i;
            v[u][i] = (part < S && col < vdim) ? po[(size_t)part * vdim + col] : 0.f;
        }
    }
    const float M = pb_warp_max(ms);
    const float ws = ms == -INFINITY ? 0.f : exp2f(ms - M);
    const float L = pb_warp_sum(ws * ls);
    const float share = L > 0.f ? ws / L : 0.f;               // of part `lane`
    float a[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const float wgt = __shfl_sync(0xffffffffu, share, (w + 4 * u) & 31);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = fmaf(w + 4 * u < S ? wgt : 0.f, v[u][i], a[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[c][w][lane + 32 * i] = a[i];
    __syncthreads();
    if (threadIdx.x >= 32) return;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int col = lane + 32 * i;
        const float a0 = (acc_s[0][0][col] + acc_s[0][1][col]) + (acc_s[0][2][col] + acc_s[0][3][col]);
        const float a1 = (acc_s[1][0][col] + acc_s[1][1][col]) + (acc_s[1][2][col] + acc_s[1][3][col]);
        a[i] = col < vdim ? a0 - p.lambda * a1 : 0.f;
        ss += a[i] * a[i];
    }
    ss = pb_warp_sum(ss);
    const float f = p.out_scale / sqrtf(ss / (float)vdim + p.norm_eps);
    __nv_bfloat16* dst = p.out + ((size_t)tok * p.n_heads + head) * vdim;
    const __nv_bfloat16* gt = p.gate ? p.gate + (size_t)tok * p.gate_stride + (size_t)head * vdim : nullptr;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int col = lane + 32 * i;
        if (col < vdim) {
            float x = a[i] * f;
            if (gt) x *= 1.0f / (1.0f + expf(-__bfloat162float(gt[col])));
            dst[col] = __float2bfloat16_rn(x);
        }
    }
}

static size_t diff_attention_smem(int dim, int vdim, int stages) {
    const size_t loop = ((size_t)2 * 64 * (dim + 8) + (size_t)stages * (2 * 64 * (dim + 8) + 64 * (vdim + 8))) * 2;
    const size_t epi = (size_t)64 * (vdim + 4) * 4;
    return loop > epi ? loop : epi;
}

// Whether the tensor-core kernel takes the shape: sizes in multiples of 16 up to 256, at most 64 query heads per
// key/value head, projection rows whose heads start on 16-byte boundaries.
PB_API int pb_diff_attention_tc_supported(int n_heads, int n_kv_heads, int dim, int vdim, long long q_stride) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads || n_heads / n_kv_heads > 64) return 0;
    if (dim < 16 || dim > 256 || dim % 16 || vdim < 16 || vdim > 256 || vdim % 16) return 0;
    if (q_stride % 8) return 0;
    return 1;
}

// Partial sums a decode step leaves per (token, head, map) when its keys are cut into n_splits ranges: with sixteen query
// heads per key/value head at most, the four warps of a map leave one each per range.
static int diff_attention_parts(int n_heads, int n_kv_heads, int n_splits) { return n_heads / n_kv_heads <= 16 ? 4 * n_splits : n_splits; }

PB_API int pb_diff_attention_tc_max_splits(int n_heads, int n_kv_heads) { return n_heads / n_kv_heads <= 16 ? 8 : 32; }

PB_API long long pb_diff_attention_tc_scratch_floats(int n_tokens, int n_heads, int n_kv_heads, int vdim, int n_splits) {
    const int parts = diff_attention_parts(n_heads, n_kv_heads, n_splits);
    return parts > 1 ? (long long)n_tokens * n_heads * 2 * parts * (vdim + 2) : 0;
}

// tile_seq null: a tile per token (decoded tokens), n_tiles = n_tokens, and n_splits blocks per tile with `scratch`
// holding pb_diff_attention_tc_scratch_floats floats; else the tiles of prompt portions (64 / group tokens each) and
// n_splits = 1.
PB_API int pb_diff_attention_tc_bf16(const void* q, long long q_stride, const void* gate, long long gate_stride, const void* k_pages,
                                     const void* v_pages, void* out, const int32_t* block_table, int table_stride,
                                     const int32_t* positions, const int32_t* token_row, const int32_t* cu_q,
                                     const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size, int num_pages,
                                     int n_tokens, int n_heads, int n_kv_heads, int dim, int vdim, float scale, float temp_coef,
                                     int temp_every, float lambda, float norm_eps, float out_scale, int window, int k_swizzle,
                                     int v_swizzle, int n_splits, int split_weights, float* scratch, int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_diff_attention_tc_supported(n_heads, n_kv_heads, dim, vdim, q_stride), "diff_attention_tc: shape not taken "
               "(heads %d over %d, dim %d, vdim %d, row stride %lld)", n_heads, n_kv_heads, dim, vdim, q_stride);
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0 && temp_every > 0, "diff_attention_tc: bad cache geometry or temperature step");
    PB_REQUIRE(q && k_pages && v_pages && out && block_table && positions && token_row, "diff_attention_tc: null pointer");
    PB_REQUIRE(pb_aligned(q, 16) && pb_aligned(k_pages, 16) && pb_aligned(v_pages, 16) && pb_aligned(out, 4),
               "diff_attention_tc: q and the pages must be 16-byte aligned");
    PB_REQUIRE((tile_seq == nullptr) == (tile_tok0 == nullptr) && (tile_seq == nullptr || cu_q != nullptr), "diff_attention_tc: half a plan");
    const bool dec = tile_seq == nullptr && n_heads / n_kv_heads <= 16;       // decoded tokens whose rows fit one warp
    const int n_parts = dec ? diff_attention_parts(n_heads, n_kv_heads, n_splits) : n_splits;
    PB_REQUIRE(n_splits >= 1 && n_parts <= 32 && (n_parts == 1 || (tile_seq == nullptr && scratch != nullptr)),
               "diff_attention_tc: %d key ranges, %d partial sums", n_splits, n_parts);
    if (n_tiles == 0) return 0;
    DiffAttnParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
    p.gate = (const __nv_bfloat16*)gate; p.gate_stride = gate_stride;
    p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages; p.out = (__nv_bfloat16*)out;
    p.block_table = block_table; p.positions = positions; p.token_row = token_row;
    p.cu_q = cu_q; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0;
    p.n_splits = n_splits;
    p.split_weights = split_weights;
    p.part_o = scratch;
    p.n_parts = n_parts;
    p.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * 2 * n_parts * vdim : nullptr;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.dim = dim; p.vdim = vdim; p.group = n_heads / n_kv_heads; p.window = window;
    p.k_swizzle = k_swizzle; p.v_swizzle = v_swizzle;
    p.scale_log2 = scale * 1.4426950408889634f; p.temp_coef = temp_coef; p.temp_every = temp_every;
    p.lambda = lambda; p.norm_eps = norm_eps; p.out_scale = out_scale; p.status = status;
    p.stages = diff_attention_smem(dim, vdim, 2) <= 200 * 1024 ? 2 : 1;
    const size_t smem = diff_attention_smem(dim, vdim, p.stages);
    dim3 grid(n_tiles, n_kv_heads, n_splits);
    PB_REQUIRE(grid.y < 65536, "diff_attention_tc: too many key/value heads");
#define DA_LAUNCH_K(NVT, KST, DECT)                                                                                              \
    do {                                                                                                                         \
        static bool set_##NVT##_##KST##_##DECT = false;                                                                          \
        if (!set_##NVT##_##KST##_##DECT) {                                                                                       \
            cudaFuncSetAttribute(diff_attention_mma_kernel<NVT, KST, DECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); \
            set_##NVT##_##KST##_##DECT = true;                                                                                   \
        }                                                                                                                        \
        pb_launch(diff_attention_mma_kernel<NVT, KST, DECT>, grid, dim3(256), smem, stream, p);                                  \
    } while (0)
#define DA_LAUNCH(NVT)                                 \
    do {                                               \
        if (dec) DA_LAUNCH_K(NVT, 0, true);            \
        else if (dim == 64) DA_LAUNCH_K(NVT, 4, false); \
        else if (dim == 128) DA_LAUNCH_K(NVT, 8, false); \
        else DA_LAUNCH_K(NVT, 0, false);               \
    } while (0)
    if (vdim <= 32) DA_LAUNCH(2);
    else if (vdim <= 64) DA_LAUNCH(4);
    else if (vdim <= 96) DA_LAUNCH(6);
    else if (vdim <= 128) DA_LAUNCH(8);
    else DA_LAUNCH(16);
#undef DA_LAUNCH_K
#undef DA_LAUNCH
    PB_CHECK_LAUNCH("diff_attention_tc");
    if (n_parts > 1) {
        const long long items = (long long)n_tokens * n_heads;
        PB_REQUIRE(items < (1ll << 31), "diff_attention_tc: too many rows");
        pb_launch(diff_attention_merge_kernel, dim3((unsigned)items), dim3(256), 0, stream, p);
        PB_CHECK_LAUNCH("diff_attention_merge");
    }
    return 0;
}
