// Attention over a shared latent row per token on tensor cores (bfloat16 operands, float32
// accumulation, scores and softmax in 32-bit).
//
// With the queries folded (see latent_attention.cu) every head reads the same key rows, and
// the first `rank` numbers of a row are also its value: a tile's M rows are (token, head)
// pairs, all heads of up to 64 / heads consecutive tokens of one request, and a block of 64
// keys brought to shared memory once serves them all, as key and as value.
//
// One CTA = one work item (some consecutive tokens of a request, all heads) x one range of
// keys (a multiple of 64 absolute positions).  Its warps are WARPS / kw row tiles of 16 rows
// times kw parts of every key block:
//   kw = 1, 8 warps  prompt portions: 128 rows, each warp walks all keys for its 16 rows
//   kw = 4, 4 warps  single tokens with up to 16 heads: the warps share the rows and split
//                    the keys; their results are joined in shared memory (warp order)
// S = Q K^T and O += P V are mma.sync m16n8k16; Q and K fragments come by ldmatrix, V fragments
// by ldmatrix.trans from the same rows, P stays in registers.  Key blocks are double
// buffered with cp.async.  Every key range leaves a partial result (running maximum, sum,
// unnormalised rows) in a workspace; a second kernel joins a row's partials in a fixed
// order, adds the optional sink to the denominator and normalises.
// Which keys meet in which partial depends on absolute positions only, so a row's result
// does not depend on the rest of the batch.
#include "common.cuh"

namespace {
constexpr int LM_ROWS = 128;         // most rows of a work item (8 warps, kw = 1)
constexpr int LM_KEYS = 64;
constexpr int LM_MAX_PARTS = 32;     // most key ranges of a row (a lane each in the join)

struct LmArgs {
    const __nv_bfloat16* qa;      // [T, heads, D]
    const __nv_bfloat16* cache;   // [pages, 1, page_size, D]
    const int* block_table;       // [requests, max_pages]
    const int* seq_of_token;
    const int* positions;
    const int* item_row0;         // first token row of every item
    const int* item_tokens;       // tokens of every item, or null: one each
    const int* item_count;        // device-side count, or null
    float* out;                   // [T, heads, rank]: written here when a row has one key range
    __nv_bfloat16* out_bf;        // instead of out: bfloat16, times sigmoid(gate[t, h])
    const float* gate;            // [T, gate_ld], head h at column h; or null
    long gate_ld;
    const float* sinks;           // [heads] or null
    const float* freq;            // [rot_dims / 2], or null: the queries come rotated
    int rot_dims;                 // how many of the rot_dim numbers the rotation covers
    float* ws_o;                  // [(item * ws_rows + row) * parts + part][rank]
    float* ws_ml;                 // [(item * ws_rows + row) * parts + part][2]
    int ws_rows;                  // rows an item has room for in the workspace
    int n_items, heads, rank, rot_dim, page_size, max_pages, num_pages, window, split_keys, parts,
        kw;
    float scale;
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                         // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// What a row's unnormalised sums are multiplied by when its keys were one range: 1 over the
// softmax's denominator, which also holds exp(sink) when the head has a sink.
__device__ __forceinline__ float lm_finish(float m, float l, const float* sinks, int h) {
    const float sk = sinks ? sinks[h] : -INFINITY;
    const float top = fmaxf(m, sk);
    if (top == -INFINITY) return 0.0f;
    const float f = (m == -INFINITY) ? 0.0f : expf(m - top);
    const float denom = l * f + (sinks ? expf(sk - top) : 0.0f);
    return denom > 0.0f ? f / denom : 0.0f;
}

// The factor of a finished row's gate (1 without one), and the store of finished numbers in
// the output's type.
__device__ __forceinline__ float lm_gate(const float* gate, long gate_ld, int t, int h) {
    return gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_ld + h])) : 1.0f;
}

// NT_O: value tiles of 8 coordinates a warp accumulates (rank <= 8 * NT_O).
template <int NT_O, int WARPS>
__global__ void __launch_bounds__(32 * WARPS)
latent_mma_kernel(LmArgs a) {
    constexpr int LM_THREADS = 32 * WARPS;
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int D = a.rank + a.rot_dim, LD = D + 8;         // (+8: rows 16 bytes apart in the banks)
    const int q_rows = 16 * WARPS / a.kw;                 // rows of the item's tile
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lm_smem);
    __nv_bfloat16* kbuf[2] = {qs + q_rows * LD, qs + (q_rows + LM_KEYS) * LD};
    prb_grid_launch_dependents();          // (a product that follows may set itself up meanwhile)
    const int item = blockIdx.x, split = blockIdx.y;
    if (item >= a.n_items || (a.item_count != nullptr && item >= *a.item_count)) return;
    const int t0 = a.item_row0[item];
    const int ntok = a.item_tokens ? a.item_tokens[item] : 1;
    if (ntok <= 0) return;
    const int b = a.seq_of_token[t0];
    if (b < 0) return;
    const int pos0 = a.positions[t0], pos_max = pos0 + ntok - 1;
    const int k_begin = split * a.split_keys;
    if (k_begin > pos_max) return;
    if (pos0 < 0 || pos_max >= a.max_pages * a.page_size) {
        if (threadIdx.x == 0 && split == 0)
            prb_set_status(a.status, PRB_S_POSITION_RANGE, t0, pos_max, a.max_pages * a.page_size);
        return;
    }
    const int k_end = min(k_begin + a.split_keys, pos_max + 1);
    const int lo_min = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int kb_first = max(k_begin, lo_min) / LM_KEYS * LM_KEYS;
    const int nrows = min(min(ntok * a.heads, q_rows), a.ws_rows);
    const int* table = a.block_table + (size_t)b * a.max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int chunks = D / 8;                              // 16-byte pieces of a row

    // the queries of the item: rows t0 * heads .. of qa, contiguous
    {
        const __nv_bfloat16* src = a.qa + (size_t)t0 * a.heads * D;
        for (int c = tid; c < q_rows * chunks; c += LM_THREADS) {
            const int r = c / chunks, k = c - r * chunks;
            cp_async16(qs + r * LD + k * 8, src + (size_t)r * D + k * 8, r < nrows);
        }
    }
    // a thread copies pieces of ONE key row of a block: one look-up in the block table, then
    // copies that do not wait for one another
    constexpr int TPR = LM_THREADS / LM_KEYS;              // threads per key row
    const int lrow = tid / TPR, lsub = tid - lrow * TPR;
    // (the page of a block's row is asked for a block ahead of its copies, so that the copies
    // do not wait for the block table)
    auto page_of = [&](int kb) {
        const int j = kb + lrow;
        return j < k_end ? table[j / a.page_size] : -1;
    };
    auto load_keys = [&](int kb, __nv_bfloat16* dst, int page) {
        const int j = kb + lrow;
        bool ok = j < k_end;
        const __nv_bfloat16* src = a.cache;
        if (ok) {
            if (page < 0 || page >= a.num_pages) {
                if (lsub == 0 && j >= lo_min) prb_set_status(a.status, PRB_S_PAGE_RANGE, t0, j, page);
                ok = false;
            } else {
                src = a.cache + ((size_t)page * a.page_size + (j % a.page_size)) * D;
            }
        }
        for (int k = lsub; k < chunks; k += TPR)
            cp_async16(dst + lrow * LD + k * 8, ok ? src + k * 8 : src, ok);
    };
    load_keys(kb_first, kbuf[0], page_of(kb_first));
    cp_async_commit();
    int page_next = page_of(kb_first + LM_KEYS);

    const int kw = a.kw, mt = warp / kw, kq = warp - mt * kw;
    const int kpw = LM_KEYS / kw, nts = kpw / 8;           // keys and score tiles of this warp a block
    const bool active = mt * 16 < nrows;
    const int row0 = mt * 16 + g, row1 = row0 + 8;
    const int p0 = row0 < nrows ? pos0 + row0 / a.heads : -1;          // -1: sees nothing
    const int p1 = row1 < nrows ? pos0 + row1 / a.heads : -1;
    const int lo0 = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
    const int lo1 = a.window > 0 ? max(0, p1 - a.window + 1) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    int buf = 0;
    for (int kb = kb_first; kb < k_end; kb += LM_KEYS, buf ^= 1) {
        if (kb + LM_KEYS < k_end) load_keys(kb + LM_KEYS, kbuf[buf ^ 1], page_next);
        cp_async_commit();
        page_next = page_of(kb + 2 * LM_KEYS);
        cp_async_wait<1>();
        __syncthreads();
        if (a.freq != nullptr && kb == kb_first) {
            // the queries arrived as their product left them: the last rot_dim numbers of a row
            // are rotated here by the row's position (pairs i, i + rot_dims / 2; 32-bit)
            const int half = a.rot_dims / 2;
            for (int e = tid; e < nrows * half; e += LM_THREADS) {
                const int r = e / half, i = e - r * half;
                __nv_bfloat16* p = qs + r * LD + a.rank + i;
                const float u = __bfloat162float(p[0]), v = __bfloat162float(p[half]);
                float sn, cs;
                sincosf((float)(pos0 + r / a.heads) * a.freq[i], &sn, &cs);
                p[0] = __float2bfloat16_rn(u * cs - v * sn);
                p[half] = __float2bfloat16_rn(v * cs + u * sn);
            }
            __syncthreads();
        }
        const __nv_bfloat16* ks = kbuf[buf];
        if (active) {
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll 2
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t qa[4];
                ldsm_x4(qa, qs + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 +
                                (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    if (np * 2 < nts) {
                        uint32_t kf[4];
                        const int key = kq * kpw + np * 16 + (lane & 7) + (lane >> 4) * 8;
                        ldsm_x4(kf, ks + key * LD + kk * 16 + ((lane >> 3) & 1) * 8);
                        mma_bf16(s[2 * np], qa, kf[0], kf[1]);
                        mma_bf16(s[2 * np + 1], qa, kf[2], kf[3]);
                    }
                }
            }
            // scale, mask, running maximum
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (nt < nts) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = kb + kq * kpw + nt * 8 + 2 * tg + (e & 1);
                        const int p = e < 2 ? p0 : p1, lo = e < 2 ? lo0 : lo1;
                        float v = s[nt][e] * a.scale;
                        if (key > p || key < lo || key < k_begin || key >= k_end) v = -INFINITY;
                        s[nt][e] = v;
                        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                    }
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            const float c0 = (m0 == -INFINITY) ? 0.0f : expf(m0 - n0);
            const float c1 = (m1 == -INFINITY) ? 0.0f : expf(m1 - n1);
            m0 = n0;
            m1 = n1;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (nt < nts) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s[nt][e];
                        const float w = (v == -INFINITY) ? 0.0f : expf(v - (e < 2 ? n0 : n1));
                        s[nt][e] = w;
                        if (e < 2) sum0 += w; else sum1 += w;
                    }
                }
            }
            l0 = l0 * c0 + sum0;
            l1 = l1 * c1 + sum1;
#pragma unroll
            for (int i = 0; i < NT_O; ++i) {
                o[i][0] *= c0;
                o[i][1] *= c0;
                o[i][2] *= c1;
                o[i][3] *= c1;
            }
            // O += P V: the first `rank` numbers of the same rows
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                if (kk * 2 < nts) {
                    uint32_t pf[4];
                    pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                    pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                    pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                    pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                    const int key = kq * kpw + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int np = 0; np < NT_O / 2; ++np) {
                        if (np * 16 < a.rank) {
                            uint32_t vf[4];
                            ldsm_x4_trans(vf, ks + key * LD + np * 16 + (lane >> 4) * 8);
                            mma_bf16(o[2 * np], pf, vf[0], vf[1]);
                            mma_bf16(o[2 * np + 1], pf, vf[2], vf[3]);
                        }
                    }
                }
            }
        }
        __syncthreads();                                   // the buffer may be filled again
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (kw > 1) {
        // the kw warps of a row tile hold the same rows over different keys: joined in warp
        // order through the key buffers, once every thread's copies into them have landed
        __syncthreads();
        float* red_ml = reinterpret_cast<float*>(kbuf[0]);           // [WARPS][16][2]
        float* red_f = red_ml + WARPS * 16 * 2;                       // [WARPS][16]
        float* red_o = red_f + WARPS * 16;                            // [WARPS][16][rank]
        if (tg == 0) {
            red_ml[(warp * 16 + g) * 2] = m0;
            red_ml[(warp * 16 + g) * 2 + 1] = l0;
            red_ml[(warp * 16 + g + 8) * 2] = m1;
            red_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
        }
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * tg;
            if (d < a.rank) {
                *reinterpret_cast<float2*>(red_o + (size_t)(warp * 16 + g) * a.rank + d) =
                    make_float2(o[nt][0], o[nt][1]);
                *reinterpret_cast<float2*>(red_o + (size_t)(warp * 16 + g + 8) * a.rank + d) =
                    make_float2(o[nt][2], o[nt][3]);
            }
        }
        __syncthreads();
        const int tiles = WARPS / kw;
        for (int e = tid; e < tiles * 16; e += LM_THREADS) {
            const int tile = e / 16, r = e - tile * 16;
            float top = -INFINITY;
            for (int w = 0; w < kw; ++w) top = fmaxf(top, red_ml[((tile * kw + w) * 16 + r) * 2]);
            float sum = 0.0f;
            for (int w = 0; w < kw; ++w) {
                const float mw = red_ml[((tile * kw + w) * 16 + r) * 2];
                const float f = (mw == -INFINITY) ? 0.0f : expf(mw - top);
                red_f[(tile * kw + w) * 16 + r] = f;
                sum += red_ml[((tile * kw + w) * 16 + r) * 2 + 1] * f;
            }
            const int row = tile * 16 + r;
            if (row < nrows) {
                if (a.parts == 1) {                       // the only range: normalise here
                    float fin = lm_finish(top, sum, a.sinks, row % a.heads);
                    if (a.out_bf) fin *= lm_gate(a.gate, a.gate_ld, t0 + row / a.heads, row % a.heads);
                    for (int w = 0; w < kw; ++w) red_f[(tile * kw + w) * 16 + r] *= fin;
                } else {
                    const size_t slot = ((size_t)item * a.ws_rows + row) * a.parts + split;
                    a.ws_ml[slot * 2] = top;
                    a.ws_ml[slot * 2 + 1] = sum;
                }
            }
        }
        __syncthreads();
        for (int e = tid; e < tiles * 16 * a.rank; e += LM_THREADS) {
            const int row = e / a.rank, d = e - row * a.rank;
            if (row >= nrows) continue;
            const int tile = row / 16, r = row - tile * 16;
            float acc = 0.0f;
            for (int w = 0; w < kw; ++w)
                acc += red_o[(size_t)((tile * kw + w) * 16 + r) * a.rank + d] *
                       red_f[(tile * kw + w) * 16 + r];
            if (a.parts == 1 && a.out_bf)
                a.out_bf[((size_t)t0 * a.heads + row) * a.rank + d] = __float2bfloat16_rn(acc);
            else if (a.parts == 1)
                a.out[((size_t)t0 * a.heads + row) * a.rank + d] = acc;
            else
                a.ws_o[(((size_t)item * a.ws_rows + row) * a.parts + split) * a.rank + d] = acc;
        }
        return;
    }
    if (!active) return;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? row1 : row0;
        if (row >= nrows) continue;
        float* dst = nullptr;
        float fin = 1.0f;
        if (a.parts == 1) {                               // the only range: normalise here
            fin = lm_finish(half ? m1 : m0, half ? l1 : l0, a.sinks, row % a.heads);
            if (a.out_bf) {
                fin *= lm_gate(a.gate, a.gate_ld, t0 + row / a.heads, row % a.heads);
                __nv_bfloat16* bdst = a.out_bf + ((size_t)t0 * a.heads + row) * a.rank;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    const int d = nt * 8 + 2 * tg;
                    if (d < a.rank)
                        *reinterpret_cast<__nv_bfloat162*>(bdst + d) =
                            half ? __floats2bfloat162_rn(o[nt][2] * fin, o[nt][3] * fin)
                                 : __floats2bfloat162_rn(o[nt][0] * fin, o[nt][1] * fin);
                }
                continue;
            }
            dst = a.out + ((size_t)t0 * a.heads + row) * a.rank;
        } else {
            const size_t slot = ((size_t)item * a.ws_rows + row) * a.parts + split;
            if (tg == 0) {
                a.ws_ml[slot * 2] = half ? m1 : m0;
                a.ws_ml[slot * 2 + 1] = half ? l1 : l0;
            }
            dst = a.ws_o + slot * a.rank;
        }
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * tg;
            if (d < a.rank)
                *reinterpret_cast<float2*>(dst + d) =
                    half ? make_float2(o[nt][2] * fin, o[nt][3] * fin)
                         : make_float2(o[nt][0] * fin, o[nt][1] * fin);
        }
    }
}

// One warp per (item, row): joins the row's partial results in order.  Lane p holds part p's
// maximum and sum; the denominator also takes the head's sink.
__global__ void __launch_bounds__(128)
latent_merge_kernel(float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf,
                    const float* __restrict__ gate, long gate_ld, const float* __restrict__ ws_o,
                    const float* __restrict__ ws_ml, const int* __restrict__ item_row0,
                    const int* __restrict__ item_tokens, const int* __restrict__ item_count,
                    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                    const float* __restrict__ sinks, int n_items, int heads, int rank, int parts,
                    int split_keys, int ws_rows) {
    prb_grid_launch_dependents();
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int item = unit / ws_rows, row = unit - item * ws_rows;
    if (item >= n_items || (item_count != nullptr && item >= *item_count)) return;
    const int ntok = item_tokens ? item_tokens[item] : 1;
    if (row >= ntok * heads) return;
    const int t = item_row0[item] + row / heads, h = row % heads;
    float* o = out ? out + ((size_t)t * heads + h) * rank : nullptr;
    __nv_bfloat16* ob = out_bf ? out_bf + ((size_t)t * heads + h) * rank : nullptr;
    const int pos = positions[t];
    if (seq_of_token[t] < 0 || pos < 0) {
        for (int d = lane; d < rank; d += 32) {
            if (ob) ob[d] = __float2bfloat16_rn(0.0f); else o[d] = 0.0f;
        }
        return;
    }
    const int n = min(parts, pos / split_keys + 1);
    const size_t base = ((size_t)item * ws_rows + row) * parts;
    const float m = lane < n ? ws_ml[(base + lane) * 2] : -INFINITY;
    const float l = lane < n ? ws_ml[(base + lane) * 2 + 1] : 0.0f;
    const float sk = sinks ? sinks[h] : -INFINITY;
    const float top = fmaxf(prb_warp_max(m), sk);
    const float f = (m == -INFINITY) ? 0.0f : expf(m - top);
    const float denom = prb_warp_sum(l * f) + (sinks ? expf(sk - top) : 0.0f);
    float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    if (ob) inv *= lm_gate(gate, gate_ld, t, h);
    float acc[8];                                          // (rank <= 256: eight per lane)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    for (int p0 = 0; p0 < n; p0 += 4) {                    // four parts' rows in flight at once
        float v[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int d = lane + 32 * k;
                v[i][k] = (p0 + i < n && d < rank) ? ws_o[(base + p0 + i) * rank + d] : 0.0f;
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float fp = __shfl_sync(0xffffffffu, f, (p0 + i) & 31);
            if (p0 + i < n && fp != 0.0f) {
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(v[i][k], fp, acc[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int d = lane + 32 * k;
        if (d < rank) {
            if (ob) ob[d] = __float2bfloat16_rn(acc[k] * inv); else o[d] = acc[k] * inv;
        }
    }
}
}  // namespace

PRB_API int prb_latent_mma_supports(int heads, int rank, int rot_dim) {
    if (heads <= 0 || heads > LM_ROWS || rank <= 0 || rank > 256 || rank % 16 != 0 || rot_dim < 0 ||
        rot_dim % 16 != 0)
        return 0;
    const size_t smem = (size_t)(LM_ROWS + 2 * LM_KEYS) * (rank + rot_dim + 8) * sizeof(__nv_bfloat16);
    return smem <= 220 * 1024 ? 1 : 0;
}

// How the warps of a CTA share single tokens: the key parts per block (4, 2 or 1).
PRB_API int prb_latent_mma_single_kw(int heads) { return heads <= 16 ? 4 : (heads <= 32 ? 2 : 1); }
PRB_API int prb_latent_mma_rows() { return LM_ROWS; }

PRB_API int prb_latent_attention_mma(float* out, void* out_bf, const float* gate, long gate_ld,
                                     const void* qa, const void* cache,
                                     const int* block_table, const int* seq_of_token,
                                     const int* positions, const int* item_row0,
                                     const int* item_tokens, const int* item_count, int n_items,
                                     const float* sinks, float* ws_o, float* ws_ml, int heads,
                                     int rank, int rot_dim, int page_size, int max_pages,
                                     int num_pages, float scale, int window, int split_keys,
                                     int splits, int kw, int ws_rows, const float* freq,
                                     int rot_dims, int* status, cudaStream_t stream) {
    // kw = 1: 8 warps, up to 128 rows an item; kw = 4 or 2: 4 warps, 16 or 32 rows
    const int warps = kw == 1 ? 8 : 4;
    const int q_rows = 16 * warps / (kw > 0 ? kw : 1);
    if (n_items <= 0) return 0;
    if (!prb_latent_mma_supports(heads, rank, rot_dim) || page_size <= 0 || max_pages <= 0 ||
        split_keys <= 0 || split_keys % LM_KEYS != 0 || splits <= 0 || splits > 65535 ||
        (kw != 1 && kw != 2 && kw != 4) || ws_rows <= 0 || ws_rows > q_rows ||
        (item_tokens == nullptr && heads > ws_rows) || heads > q_rows || splits > LM_MAX_PARTS)
        return PRB_E_SIZE;
    if (((uintptr_t)qa) % 16 != 0 || ((uintptr_t)cache) % 16 != 0) return PRB_E_ALIGN;
    if ((out == nullptr) == (out_bf == nullptr)) return PRB_E_ARG;
    if (freq != nullptr && (rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 != 0)) return PRB_E_SIZE;
    LmArgs a{(const __nv_bfloat16*)qa, (const __nv_bfloat16*)cache, block_table, seq_of_token,
             positions, item_row0, item_tokens, item_count, out, (__nv_bfloat16*)out_bf, gate, gate_ld,
             sinks, freq, rot_dims, ws_o, ws_ml, ws_rows, n_items,
             heads, rank,
             rot_dim, page_size, max_pages, num_pages, window, split_keys, splits, kw, scale,
             status};
    const size_t smem = (size_t)(q_rows + 2 * LM_KEYS) * (rank + rot_dim + 8) * sizeof(__nv_bfloat16);
    dim3 grid(n_items, splits);
#define PRB_LM(NT, W)                                                                           \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(latent_mma_kernel<NT, W>,                                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        latent_mma_kernel<NT, W><<<grid, 32 * W, smem, stream>>>(a);                            \
    } while (0)
#define PRB_LM_RANK(W)                   \
    do {                                 \
        if (rank <= 64) PRB_LM(8, W);    \
        else if (rank <= 128) PRB_LM(16, W); \
        else if (rank <= 192) PRB_LM(24, W); \
        else PRB_LM(32, W);              \
    } while (0)
    if (warps == 8) PRB_LM_RANK(8);
    else PRB_LM_RANK(4);
#undef PRB_LM_RANK
#undef PRB_LM
    PRB_LAUNCH_CHECK();
    if (splits == 1) return 0;                 // every row had one range and is finished
    latent_merge_kernel<<<(n_items * ws_rows + 3) / 4, 128, 0, stream>>>(
        out, (__nv_bfloat16*)out_bf, gate, gate_ld, ws_o, ws_ml, item_row0, item_tokens, item_count,
        seq_of_token, positions, sinks, n_items, heads, rank, splits, split_keys, ws_rows);
    PRB_LAUNCH_CHECK();
    return 0;
}
