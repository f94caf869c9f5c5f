// Attention over a shared latent row per token on tensor cores (bfloat16 operands, float32
// accumulation, scores and softmax in 32-bit).
//
// With the queries folded (see latent_attention.cu) every head reads the same key rows, and
// the first `rank` numbers of a row are also its value: a tile's M rows are (token, head)
// pairs, all heads of up to 64 / heads consecutive tokens of one request, and a block of 64
// keys brought to shared memory once serves them all, as key and as value.
//
// One CTA = one work item (some consecutive tokens of a request, all heads) x one range of
// keys (a multiple of 64 absolute positions).  Its four warps are 4 / kw row tiles of 16 rows
// times kw parts of every key block:
//   kw = 1  prompt portions: 64 rows, each warp walks all keys for its 16 rows
//   kw = 4  single tokens with up to 16 heads: the warps share the rows and split the keys
// S = Q K^T and O += P V are mma.sync m16n8k16; Q and K fragments come by ldmatrix, V fragments
// by ldmatrix.trans from the same rows, P stays in registers.  Key blocks are double
// buffered with cp.async.  Every (warp's key part) x (key range) leaves a partial result
// (running maximum, sum, unnormalised rows) in a workspace; prb_latent_merge joins a row's
// partials in a fixed order, adds the optional sink to the denominator and normalises.
// Which keys meet in which partial depends on absolute positions only, so a row's result
// does not depend on the rest of the batch.
#include "common.cuh"

namespace {
constexpr int LM_THREADS = 128;
constexpr int LM_ROWS = 64;
constexpr int LM_KEYS = 64;

struct LmArgs {
    const __nv_bfloat16* qa;      // [T, heads, D]
    const __nv_bfloat16* cache;   // [pages, 1, page_size, D]
    const int* block_table;       // [requests, max_pages]
    const int* seq_of_token;
    const int* positions;
    const int* item_row0;         // first token row of every item
    const int* item_tokens;       // tokens of every item, or null: one each
    const int* item_count;        // device-side count, or null
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

// NT_O: value tiles of 8 coordinates a warp accumulates (rank <= 8 * NT_O).
template <int NT_O>
__global__ void __launch_bounds__(LM_THREADS)
latent_mma_kernel(LmArgs a) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int D = a.rank + a.rot_dim, LD = D + 8;         // (+8: rows 16 bytes apart in the banks)
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lm_smem);
    __nv_bfloat16* kbuf[2] = {qs + LM_ROWS * LD, qs + 2 * LM_ROWS * LD};
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
    const int nrows = min(min(ntok * a.heads, LM_ROWS), a.ws_rows);
    const int* table = a.block_table + (size_t)b * a.max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tg = lane & 3;
    const int chunks = D / 8;                              // 16-byte pieces of a row

    // the queries of the item: rows t0 * heads .. of qa, contiguous
    {
        const __nv_bfloat16* src = a.qa + (size_t)t0 * a.heads * D;
        for (int c = tid; c < LM_ROWS * chunks; c += LM_THREADS) {
            const int r = c / chunks, k = c - r * chunks;
            cp_async16(qs + r * LD + k * 8, src + (size_t)r * D + k * 8, r < nrows);
        }
    }
    auto load_keys = [&](int kb, __nv_bfloat16* dst) {
        for (int c = tid; c < LM_KEYS * chunks; c += LM_THREADS) {
            const int r = c / chunks, k = c - r * chunks;
            const int j = kb + r;
            bool ok = j < k_end;
            const __nv_bfloat16* src = a.cache;
            if (ok) {
                const int page = table[j / a.page_size];
                if (page < 0 || page >= a.num_pages) {
                    if (k == 0 && j >= lo_min) prb_set_status(a.status, PRB_S_PAGE_RANGE, t0, j, page);
                    ok = false;
                } else {
                    src = a.cache + ((size_t)page * a.page_size + (j % a.page_size)) * D + k * 8;
                }
            }
            cp_async16(dst + r * LD + k * 8, src, ok);
        }
    };
    load_keys(kb_first, kbuf[0]);
    cp_async_commit();

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
        if (kb + LM_KEYS < k_end) load_keys(kb + LM_KEYS, kbuf[buf ^ 1]);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* ks = kbuf[buf];
        if (active) {
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
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
    if (!active) return;
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int part = split * kw + kq;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? row1 : row0;
        if (row >= nrows) continue;
        const size_t slot = ((size_t)item * a.ws_rows + row) * a.parts + part;
        if (tg == 0) {
            a.ws_ml[slot * 2] = half ? m1 : m0;
            a.ws_ml[slot * 2 + 1] = half ? l1 : l0;
        }
        float* dst = a.ws_o + slot * a.rank;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            const int d = nt * 8 + 2 * tg;
            if (d < a.rank)
                *reinterpret_cast<float2*>(dst + d) =
                    half ? make_float2(o[nt][2], o[nt][3]) : make_float2(o[nt][0], o[nt][1]);
        }
    }
}

// grid (items * ws_rows): one CTA per (item, row); joins the row's partials in order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(float* __restrict__ out, const float* __restrict__ ws_o,
                    const float* __restrict__ ws_ml, const int* __restrict__ item_row0,
                    const int* __restrict__ item_tokens, const int* __restrict__ item_count,
                    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                    const float* __restrict__ sinks, int n_items, int heads, int rank, int parts,
                    int kw, int split_keys, int ws_rows) {
    const int item = blockIdx.x / ws_rows, row = blockIdx.x % ws_rows;
    if (item >= n_items || (item_count != nullptr && item >= *item_count)) return;
    const int ntok = item_tokens ? item_tokens[item] : 1;
    if (row >= ntok * heads) return;
    const int t = item_row0[item] + row / heads, h = row % heads;
    float* o = out + ((size_t)t * heads + h) * rank;
    const int pos = positions[t];
    if (seq_of_token[t] < 0 || pos < 0) {
        for (int d = threadIdx.x; d < rank; d += blockDim.x) o[d] = 0.0f;
        return;
    }
    const int n = min(parts, (pos / split_keys + 1) * kw);
    const size_t base = ((size_t)item * ws_rows + row) * parts;
    float top = sinks ? sinks[h] : -INFINITY;
    for (int p = 0; p < n; ++p) top = fmaxf(top, ws_ml[(base + p) * 2]);
    float denom = sinks ? expf(sinks[h] - top) : 0.0f;
    for (int p = 0; p < n; ++p) {
        const float m = ws_ml[(base + p) * 2];
        if (m != -INFINITY) denom += ws_ml[(base + p) * 2 + 1] * expf(m - top);
    }
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < n; ++p) {
            const float m = ws_ml[(base + p) * 2];
            if (m != -INFINITY) acc += ws_o[(base + p) * rank + d] * expf(m - top);
        }
        o[d] = denom > 0.0f ? acc / denom : 0.0f;
    }
}
}  // namespace

PRB_API int prb_latent_mma_supports(int heads, int rank, int rot_dim) {
    if (heads <= 0 || heads > LM_ROWS || rank <= 0 || rank > 256 || rank % 16 != 0 || rot_dim < 0 ||
        rot_dim % 16 != 0)
        return 0;
    const size_t smem = (size_t)3 * LM_ROWS * (rank + rot_dim + 8) * sizeof(__nv_bfloat16);
    return smem <= 200 * 1024 ? 1 : 0;
}

// How the warps of a CTA share single tokens: the key parts per block (4, 2 or 1).
PRB_API int prb_latent_mma_single_kw(int heads) { return heads <= 16 ? 4 : (heads <= 32 ? 2 : 1); }
PRB_API int prb_latent_mma_rows() { return LM_ROWS; }

PRB_API int prb_latent_attention_mma(float* out, const void* qa, const void* cache,
                                     const int* block_table, const int* seq_of_token,
                                     const int* positions, const int* item_row0,
                                     const int* item_tokens, const int* item_count, int n_items,
                                     const float* sinks, float* ws_o, float* ws_ml, int heads,
                                     int rank, int rot_dim, int page_size, int max_pages,
                                     int num_pages, float scale, int window, int split_keys,
                                     int splits, int kw, int ws_rows, int* status,
                                     cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (!prb_latent_mma_supports(heads, rank, rot_dim) || page_size <= 0 || max_pages <= 0 ||
        split_keys <= 0 || split_keys % LM_KEYS != 0 || splits <= 0 || splits > 65535 ||
        (kw != 1 && kw != 2 && kw != 4) || ws_rows <= 0 || ws_rows > LM_ROWS ||
        (item_tokens == nullptr && heads > ws_rows) || (kw > 1 && heads > 16 * (4 / kw)))
        return PRB_E_SIZE;
    if (((uintptr_t)qa) % 16 != 0 || ((uintptr_t)cache) % 16 != 0) return PRB_E_ALIGN;
    LmArgs a{(const __nv_bfloat16*)qa, (const __nv_bfloat16*)cache, block_table, seq_of_token,
             positions, item_row0, item_tokens, item_count, ws_o, ws_ml, ws_rows, n_items, heads, rank,
             rot_dim, page_size, max_pages, num_pages, window, split_keys, splits * kw, kw, scale,
             status};
    const size_t smem = (size_t)3 * LM_ROWS * (rank + rot_dim + 8) * sizeof(__nv_bfloat16);
    dim3 grid(n_items, splits);
#define PRB_LM(NT)                                                                              \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(latent_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                    \
        latent_mma_kernel<NT><<<grid, LM_THREADS, smem, stream>>>(a);                           \
    } while (0)
    if (rank <= 64) PRB_LM(8);
    else if (rank <= 128) PRB_LM(16);
    else if (rank <= 192) PRB_LM(24);
    else PRB_LM(32);
#undef PRB_LM
    PRB_LAUNCH_CHECK();
    latent_merge_kernel<<<n_items * ws_rows, 128, 0, stream>>>(
        out, ws_o, ws_ml, item_row0, item_tokens, item_count, seq_of_token, positions, sinks,
        n_items, heads, rank, splits * kw, kw, split_keys, ws_rows);
    PRB_LAUNCH_CHECK();
    return 0;
}
