// Differential attention over the paged cache: every query head runs TWO softmax attentions
// ("maps") over the same values and subtracts them,
//     o = a1 - lambda a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale    (per head, over vdim)
// with grouped key/value heads and an optional block mask: a query at position p sees keys
// floor(p / block) * block .. p (block 0: all keys 0 .. p), counted from the sequence's start.
//
// Cache: one pool per layer, one row per (token, key/value head): [k map 1 | k map 2 | v],
// 2 * dim + vdim numbers, so a key's two maps and its value come with one page look-up.
//
// diff_prepare: a CTA per token.  Reads the fused projection's 32-bit result, turns the first
// rot_dims coordinates of every map of q and k by the token's position (rotate-half layout,
// angles in 32-bit), leaves q in 32-bit beside the step and writes the token's cache rows.
//
// diff_attention: a CTA per (token, query head), 32-bit arithmetic; keys in segments of SEG
// with running maxima and sums per map.  Reduction orders depend on the visible range and the
// sizes only, never on the batch.
#include "common.cuh"

namespace {
constexpr int DA_THREADS = 128;
constexpr int DA_SEG = 256;         // keys scored at a time
constexpr int DA_MAX_V = 4;         // value coordinates a thread owns at most (vdim <= 512)

template <typename C>
__global__ void diff_prepare_kernel(float* __restrict__ q_out, C* __restrict__ cache,
                                    const float* __restrict__ proj, long ld, int q_col, int k_col,
                                    int v_col, const int* __restrict__ slots,
                                    const int* __restrict__ positions, const float* __restrict__ freq,
                                    int n_tokens, int heads, int kv_heads, int dim, int vdim,
                                    int rot_dims, int page_size, int num_pages, int* status) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    const int units = half + (dim - rot_dims);       // per map: pairs, then coordinates that stay
    // queries: heads * 2 maps
    float* qo = q_out + (size_t)t * heads * 2 * dim;
    for (int u = threadIdx.x; u < heads * 2 * units; u += blockDim.x) {
        const int m = u / units, w = u - m * units;
        const float* src = row + q_col + m * dim;
        float* dst = qo + m * dim;
        if (w < half) {
            float sn, cs;
            sincosf(pos * freq[w], &sn, &cs);
            const float a = src[w], b = src[w + half];
            dst[w] = a * cs - b * sn;
            dst[w + half] = b * cs + a * sn;
        } else {
            const int i = w - half + rot_dims;
            dst[i] = src[i];
        }
    }
    if (slots == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
        if (threadIdx.x == 0) prb_set_status(status, PRB_S_SLOT_RANGE, t, slot, num_pages);
        return;
    }
    const int rowlen = 2 * dim + vdim;
    for (int u = threadIdx.x; u < kv_heads * 2 * units; u += blockDim.x) {
        const int m = u / units, w = u - m * units;          // m = kv head * 2 + map
        const int g = m >> 1;
        const float* src = row + k_col + m * dim;
        C* dst = cache + (((size_t)page * kv_heads + g) * page_size + off) * rowlen + (m & 1) * dim;
        if (w < half) {
            float sn, cs;
            sincosf(pos * freq[w], &sn, &cs);
            const float a = src[w], b = src[w + half];
            dst[w] = prb_from_float<C>(a * cs - b * sn);
            dst[w + half] = prb_from_float<C>(b * cs + a * sn);
        } else {
            const int i = w - half + rot_dims;
            dst[i] = prb_from_float<C>(src[i]);
        }
    }
    for (int u = threadIdx.x; u < kv_heads * vdim; u += blockDim.x) {
        const int g = u / vdim, j = u - g * vdim;
        cache[(((size_t)page * kv_heads + g) * page_size + off) * rowlen + 2 * dim + j] =
            prb_from_float<C>(row[v_col + u]);
    }
}

template <typename C, typename O>
__global__ void __launch_bounds__(DA_THREADS)
diff_attention_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ q,
                      const C* __restrict__ cache, const int* __restrict__ block_table,
                      const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                      int n_tokens, int heads, int kv_heads, int dim, int vdim, int page_size,
                      int max_pages, int num_pages, int block, float scale, float lambda,
                      float eps, float out_scale, int* status) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    float* qs = smem;                        // [2 * dim]
    float* w1 = qs + 2 * dim;                // [DA_SEG] weights of map 1
    float* w2 = w1 + DA_SEG;                 // [DA_SEG]
    float* part = w2 + DA_SEG;               // [DA_THREADS * 2]
    prb_grid_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    if (t >= n_tokens) return;
    const int b = seq_of_token[t];
    const int pos = positions[t];
    O* o = out + (size_t)t * out_ld + (size_t)h * vdim;
    if (b < 0 || pos < 0 || pos >= max_pages * page_size) {
        if (b >= 0 && threadIdx.x == 0)
            prb_set_status(status, PRB_S_POSITION_RANGE, t, pos, max_pages * page_size);
        for (int j = threadIdx.x; j < vdim; j += blockDim.x) o[j] = prb_from_float<O>(0.0f);
        return;
    }
    const int lo = block > 0 ? (pos / block) * block : 0;
    const int n = pos - lo + 1;
    const int g = h / (heads / kv_heads);
    const int rowlen = 2 * dim + vdim;
    const int* table = block_table + (size_t)b * max_pages;
    const float* qp = q + ((size_t)t * heads + h) * 2 * dim;
    for (int i = threadIdx.x; i < 2 * dim; i += blockDim.x) qs[i] = qp[i];

    // thread (kg, j): value coordinates j, j + vthreads, ... of keys kg, kg + kgroups, ...
    const int vthreads = vdim < DA_THREADS ? vdim : DA_THREADS;
    const int kgroups = DA_THREADS / vthreads;
    const int vj = threadIdx.x % vthreads, kg = threadIdx.x / vthreads;
    const bool vlive = kg < kgroups;
    float acc1[DA_MAX_V], acc2[DA_MAX_V];
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) acc1[x] = acc2[x] = 0.0f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.0f, l2 = 0.0f;
    __syncthreads();

    for (int s0 = 0; s0 < n; s0 += DA_SEG) {
        const int ns = min(DA_SEG, n - s0);
        float mx1 = -INFINITY, mx2 = -INFINITY;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const int j = lo + s0 + i;
            const int page = table[j / page_size];
            float s1 = -INFINITY, s2 = -INFINITY;
            if (page < 0 || page >= num_pages) {
                prb_set_status(status, PRB_S_PAGE_RANGE, t, j, page);
            } else {
                const C* kp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen;
                float a1 = 0.0f, a2 = 0.0f;
                for (int d = 0; d < dim; ++d) {
                    a1 = fmaf(qs[d], prb_to_float<C>(kp[d]), a1);
                    a2 = fmaf(qs[dim + d], prb_to_float<C>(kp[dim + d]), a2);
                }
                s1 = a1 * scale;
                s2 = a2 * scale;
            }
            w1[i] = s1;
            w2[i] = s2;
            mx1 = fmaxf(mx1, s1);
            mx2 = fmaxf(mx2, s2);
        }
        mx1 = prb_block_max(mx1, scratch);
        mx2 = prb_block_max(mx2, scratch);
        const float n1 = fmaxf(m1, mx1), n2 = fmaxf(m2, mx2);
        // (a segment whose keys are all missing leaves the running state as it is)
        const float f1 = (n1 == -INFINITY) ? 1.0f : expf(m1 - n1);
        const float f2 = (n2 == -INFINITY) ? 1.0f : expf(m2 - n2);
        float sum1 = 0.0f, sum2 = 0.0f;
        for (int i = threadIdx.x; i < ns; i += blockDim.x) {
            const float e1 = (w1[i] == -INFINITY) ? 0.0f : expf(w1[i] - n1);
            const float e2 = (w2[i] == -INFINITY) ? 0.0f : expf(w2[i] - n2);
            w1[i] = e1;
            w2[i] = e2;
            sum1 += e1;
            sum2 += e2;
        }
        sum1 = prb_block_sum(sum1, scratch);
        sum2 = prb_block_sum(sum2, scratch);
        __syncthreads();                         // the weights are written
        l1 = l1 * f1 + sum1;
        l2 = l2 * f2 + sum2;
        m1 = n1;
        m2 = n2;
        if (vlive) {
#pragma unroll
            for (int x = 0; x < DA_MAX_V; ++x) {
                acc1[x] *= f1;
                acc2[x] *= f2;
            }
            for (int i = kg; i < ns; i += kgroups) {
                const float e1 = w1[i], e2 = w2[i];
                if (e1 == 0.0f && e2 == 0.0f) continue;
                const int j = lo + s0 + i;
                const int page = table[j / page_size];
                if (page < 0 || page >= num_pages) continue;
                const C* vp = cache + (((size_t)page * kv_heads + g) * page_size + (j % page_size)) * rowlen + 2 * dim;
#pragma unroll
                for (int x = 0; x < DA_MAX_V; ++x) {
                    const int jj = vj + x * vthreads;
                    if (jj < vdim) {
                        const float v = prb_to_float<C>(vp[jj]);
                        acc1[x] = fmaf(e1, v, acc1[x]);
                        acc2[x] = fmaf(e2, v, acc2[x]);
                    }
                }
            }
        }
        __syncthreads();                         // before the next segment overwrites the weights
    }

    // join the key groups in group order, combine the maps, unit RMS over the head
    float mine[DA_MAX_V];
    float ss = 0.0f;
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) {
        part[threadIdx.x * 2] = acc1[x];
        part[threadIdx.x * 2 + 1] = acc2[x];
        __syncthreads();
        mine[x] = 0.0f;
        const int jj = vj + x * vthreads;
        if (kg == 0 && jj < vdim) {
            float t1 = 0.0f, t2 = 0.0f;
            for (int gg = 0; gg < kgroups; ++gg) {
                t1 += part[(gg * vthreads + vj) * 2];
                t2 += part[(gg * vthreads + vj) * 2 + 1];
            }
            const float a1 = l1 > 0.0f ? t1 / l1 : 0.0f;
            const float a2 = l2 > 0.0f ? t2 / l2 : 0.0f;
            mine[x] = a1 - lambda * a2;
            ss = fmaf(mine[x], mine[x], ss);
        }
        __syncthreads();
    }
    ss = prb_block_sum(ss, scratch);
    const float inv = out_scale / sqrtf(ss / (float)vdim + eps);
#pragma unroll
    for (int x = 0; x < DA_MAX_V; ++x) {
        const int jj = vj + x * vthreads;
        if (kg == 0 && jj < vdim) o[jj] = prb_from_float<O>(mine[x] * inv);
    }
}
}  // namespace

PRB_API int prb_diff_prepare(float* q_out, void* cache, const float* proj, long ld, int q_col,
                             int k_col, int v_col, const int* slots, const int* positions,
                             const float* freq, int n_tokens, int heads, int kv_heads, int dim,
                             int vdim, int rot_dims, int page_size, int num_pages, int cache_dtype,
                             int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rot_dims < 0 || rot_dims > dim ||
        rot_dims % 2 != 0 || page_size <= 0)
        return PRB_E_SIZE;
    const int work = heads * 2 * dim;
    const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
    if (cache_dtype == PRB_F32)
        diff_prepare_kernel<float><<<n_tokens, threads, 0, stream>>>(
            q_out, (float*)cache, proj, ld, q_col, k_col, v_col, slots, positions, freq, n_tokens,
            heads, kv_heads, dim, vdim, rot_dims, page_size, num_pages, status);
    else if (cache_dtype == PRB_BF16)
        diff_prepare_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            q_out, (__nv_bfloat16*)cache, proj, ld, q_col, k_col, v_col, slots, positions, freq,
            n_tokens, heads, kv_heads, dim, vdim, rot_dims, page_size, num_pages, status);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_diff_attention(void* out, long out_ld, const float* q, const void* cache,
                               const int* block_table, const int* seq_of_token,
                               const int* positions, int n_tokens, int heads, int kv_heads, int dim,
                               int vdim, int page_size, int max_pages, int num_pages, int block,
                               float scale, float lambda, float eps, float out_scale,
                               int cache_dtype, int out_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 ||
        vdim <= 0 || vdim > DA_THREADS * DA_MAX_V || page_size <= 0 || max_pages <= 0 || block < 0)
        return PRB_E_SIZE;
    const size_t smem = (size_t)(2 * dim + 2 * DA_SEG + 2 * DA_THREADS) * sizeof(float);
    if (smem > 48 * 1024) return PRB_E_SIZE;
    dim3 grid(n_tokens, heads);
#define DIFF(CT, OT)                                                                            \
    diff_attention_kernel<CT, OT><<<grid, DA_THREADS, smem, stream>>>(                          \
        (OT*)out, out_ld, q, (const CT*)cache, block_table, seq_of_token, positions, n_tokens,   \
        heads, kv_heads, dim, vdim, page_size, max_pages, num_pages, block, scale, lambda, eps, \
        out_scale, status)
    if (cache_dtype == PRB_F32 && out_dtype == PRB_F32) DIFF(float, float);
    else if (cache_dtype == PRB_BF16 && out_dtype == PRB_BF16) DIFF(__nv_bfloat16, __nv_bfloat16);
    else return PRB_E_DTYPE;
#undef DIFF
    PRB_LAUNCH_CHECK();
    return 0;
}
