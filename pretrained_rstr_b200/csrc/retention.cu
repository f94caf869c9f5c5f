// Retention: linear attention with a fixed decay per head and a running state per request,
//     S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S: [dim, vdim], 32-bit)
// with rotary positions (rotate-half layout, the first rot_dims coordinates) on q and k and
// k scaled by `k_scale` after the rotation.  Everything that enters the recurrence is 32-bit.
//
// retention_scan: one CTA per (chunk of value columns, head, request).  A column of S is
// independent of the others, so columns are spread over CTAs and over the threads of a CTA; a
// column's `dim` numbers are spread over R neighbouring lanes (NI numbers a lane, in
// registers) and the dot with q is closed with R - 1 shuffles.  The CTA walks its request's
// tokens of the step in order, a block of tokens at a time: q and k of the block (rotated
// beforehand, for all tokens at once, by retention_rotate) are staged in shared memory by all
// threads, then every thread runs the recurrence over the block.  The state comes from the request's slot (zero at position 0) and goes back
// there after the last token, so a prompt may be cut anywhere and a decoded token is the
// same kernel with one token.  The order of every sum depends on dim and vdim only.
//
// retention_finish: a warp per (token, head): unit root-mean-square over the head's vdim
// values, times silu(gate), written in the activation type.
#include "common.cuh"

namespace {
constexpr int RET_BLOCK = 16;       // tokens staged at a time
// State numbers a lane holds per column: 4 for heads of up to 128 (a column over up to 32
// lanes: many short chains, which is what hides the recurrence's latency), 16 beyond.

struct ScanArgs {
    float* o_raw;             // [T, heads * vdim]
    const float* proj;        // [T, ld]: q at q_col, k at k_col (heads * dim each), v at v_col
    long ld;
    int q_col, k_col, v_col;
    float* state;             // [slots, heads, vdim, dim]
    const int* q_start;       // [requests + 1]
    const int* state_slot;    // [requests]
    const int* positions;     // [T]
    const float* decay;       // [heads]
    int n_tokens, n_slots, heads, dim, vdim, cols, lanes;   // lanes = R
    int* status;
    int n_requests, seg_len;  // segments (see below); seg_len 0: none
    float* seg_own;           // [segments, heads, vdim, dim]: pass 1's sums
    float* seg_start;         // [segments, heads, vdim, dim]: the states at the segments' starts
};

// q and k of every token of the step, in place in the projection's 32-bit result: the first
// rot_dims coordinates of every head turned by the token's position (rotate-half layout), k
// times k_scale afterwards.  A CTA per token.
__global__ void retention_rotate_kernel(float* __restrict__ proj, long ld, int q_col, int k_col,
                                        const int* __restrict__ positions,
                                        const float* __restrict__ freq, int n_tokens, int heads,
                                        int dim, int rot_dims, float k_scale) {
    prb_grid_launch_dependents();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    float* row = proj + (size_t)t * ld;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    const int units = half + (dim - rot_dims);
    for (int u = threadIdx.x; u < heads * units; u += blockDim.x) {
        const int h = u / units, w = u - h * units;
        float* qr = row + q_col + h * dim;
        float* kr = row + k_col + h * dim;
        if (w < half) {
            float sn, cs;
            sincosf(pos * freq[w], &sn, &cs);
            const float q0 = qr[w], q1 = qr[w + half], k0 = kr[w], k1 = kr[w + half];
            qr[w] = q0 * cs - q1 * sn;
            qr[w + half] = q1 * cs + q0 * sn;
            kr[w] = (k0 * cs - k1 * sn) * k_scale;
            kr[w + half] = (k1 * cs + k0 * sn) * k_scale;
        } else {
            const int i = w - half + rot_dims;
            kr[i] *= k_scale;
        }
    }
}

// Long portions are cut into segments of `seg_len` tokens that run side by side:
//   pass 1 (MODE 1): every segment but a request's last builds, from zero, what its own tokens
//           add to the state (no queries, no outputs);
//   pass 2 (carry):  per request the states at the segments' starts, one after the other:
//           U_0 = the carried state, U_(s+1) = decay^seg_len U_s + (pass 1 of segment s);
//   pass 3 (MODE 2): every segment runs the recurrence from its U_s with outputs; a request's
//           last segment leaves the state in the request's slot.
// MODE 0 is the whole portion by one CTA from and to the slot (steps of few tokens).
// Segment z of the launch is segment s of request b: requests' segments are numbered in
// request order (a CTA finds its own by walking q_start).
__device__ __forceinline__ bool find_segment(const int* q_start, int n_requests, int seg_len, int z,
                                             int& b, int& s, int& nseg) {
    int base = 0;
    for (b = 0; b < n_requests; ++b) {
        const int n = q_start[b + 1] - q_start[b];
        nseg = n > 0 ? (n + seg_len - 1) / seg_len : 0;
        if (z < base + nseg) {
            s = z - base;
            return true;
        }
        base += nseg;
    }
    return false;
}

template <int RET_NI, int MODE>
__global__ void retention_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float smem[];
    prb_grid_launch_dependents();
    const int chunk = blockIdx.x, h = blockIdx.y;
    int b = blockIdx.z, s = 0, nseg = 1;
    if (MODE != 0 && !find_segment(a.q_start, a.n_requests, a.seg_len, blockIdx.z, b, s, nseg)) return;
    int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    if (MODE != 0) {
        if (MODE == 1 && s == nseg - 1) return;      // (a last segment's own sum is never needed)
        t0 += s * a.seg_len;
        t1 = min(t1, t0 + a.seg_len);
    }
    const int R = a.lanes, dim_pad = R * RET_NI;
    float* qs = smem;                               // [RET_BLOCK][dim_pad]
    float* ks = qs + RET_BLOCK * dim_pad;           // [RET_BLOCK][dim_pad]
    float* vs = ks + RET_BLOCK * dim_pad;           // [RET_BLOCK][cols]
    const int r = threadIdx.x % R, c = threadIdx.x / R;
    const int col = chunk * a.cols + c;
    const bool live = c < a.cols && col < a.vdim;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_SLOT_RANGE, t0, slot, a.n_slots);
        return;
    }
    const size_t column = ((size_t)h * a.vdim + (live ? col : 0)) * a.dim;
    const size_t per_state = (size_t)a.heads * a.vdim * a.dim;
    float* srow = a.state + (size_t)slot * per_state + column;
    float S[RET_NI];
    {
        // where the state comes from: the slot (zero at position 0), zero, or pass 2's U
        const float* from = nullptr;
        if (MODE == 0 && a.positions[t0] > 0) from = srow;
        if (MODE == 2) from = a.seg_start + (size_t)blockIdx.z * per_state + column;
#pragma unroll
        for (int ii = 0; ii < RET_NI; ++ii) {
            const int i = r * RET_NI + ii;
            S[ii] = (live && from != nullptr && i < a.dim) ? from[i] : 0.0f;
        }
    }
    const float decay = a.decay[h];
    for (int tb = t0; tb < t1; tb += RET_BLOCK) {
        const int nb = min(RET_BLOCK, t1 - tb);
        __syncthreads();                            // the block before has been consumed
        for (int u = threadIdx.x; u < nb * a.dim; u += blockDim.x) {
            const int tok = u / a.dim, i = u - tok * a.dim;
            const float* row = a.proj + (size_t)(tb + tok) * a.ld + h * a.dim + i;
            if (MODE != 1) qs[tok * dim_pad + i] = row[a.q_col];
            ks[tok * dim_pad + i] = row[a.k_col];
        }
        for (int u = threadIdx.x; u < nb * (dim_pad - a.dim); u += blockDim.x) {
            const int tok = u / (dim_pad - a.dim), i = a.dim + u % (dim_pad - a.dim);
            qs[tok * dim_pad + i] = 0.0f;
            ks[tok * dim_pad + i] = 0.0f;
        }
        for (int u = threadIdx.x; u < nb * a.cols; u += blockDim.x) {
            const int tok = u / a.cols, cc = u - tok * a.cols;
            const int vc = chunk * a.cols + cc;
            vs[tok * a.cols + cc] = vc < a.vdim
                ? a.proj[(size_t)(tb + tok) * a.ld + a.v_col + h * a.vdim + vc] : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int tok = 0; tok < nb; ++tok) {
            const float v = c < a.cols ? vs[tok * a.cols + c] : 0.0f;
            const float4* q4 = reinterpret_cast<const float4*>(qs + tok * dim_pad + r * RET_NI);
            const float4* k4 = reinterpret_cast<const float4*>(ks + tok * dim_pad + r * RET_NI);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int g = 0; g < RET_NI / 4; ++g) {      // (sums in an order that dim alone fixes)
                const float4 kk = k4[g];
                S[4 * g + 0] = fmaf(decay, S[4 * g + 0], kk.x * v);
                S[4 * g + 1] = fmaf(decay, S[4 * g + 1], kk.y * v);
                S[4 * g + 2] = fmaf(decay, S[4 * g + 2], kk.z * v);
                S[4 * g + 3] = fmaf(decay, S[4 * g + 3], kk.w * v);
                if (MODE != 1) {
                    const float4 qq = q4[g];
                    acc[0] = fmaf(S[4 * g + 0], qq.x, acc[0]);
                    acc[1] = fmaf(S[4 * g + 1], qq.y, acc[1]);
                    acc[2] = fmaf(S[4 * g + 2], qq.z, acc[2]);
                    acc[3] = fmaf(S[4 * g + 3], qq.w, acc[3]);
                }
            }
            if (MODE != 1) {
                float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                for (int m = 1; m < R; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
                if (live && r == 0)
                    a.o_raw[(size_t)(tb + tok) * a.heads * a.vdim + h * a.vdim + col] = o;
            }
        }
    }
    // where the state goes: the slot, pass 1's own sums, or (a last segment) the slot
    float* to = nullptr;
    if (MODE == 0 || (MODE == 2 && s == nseg - 1)) to = srow;
    if (MODE == 1) to = a.seg_own + (size_t)blockIdx.z * per_state + column;
    if (live && to != nullptr) {
#pragma unroll
        for (int ii = 0; ii < RET_NI; ++ii) {
            const int i = r * RET_NI + ii;
            if (i < a.dim) to[i] = S[ii];
        }
    }
}

// Pass 2: a thread per state number of a (head, request), 1,024 numbers a CTA; the request's
// segments in order.
__global__ void retention_carry_kernel(ScanArgs a) {
    prb_grid_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) return;
    int base = 0;
    for (int bb = 0; bb < b; ++bb) {
        const int n = a.q_start[bb + 1] - a.q_start[bb];
        base += n > 0 ? (n + a.seg_len - 1) / a.seg_len : 0;
    }
    const int nseg = (t1 - t0 + a.seg_len - 1) / a.seg_len;
    const size_t per_state = (size_t)a.heads * a.vdim * a.dim;
    const size_t per_head = (size_t)a.vdim * a.dim;
    const bool carried = a.positions[t0] > 0;
    const float decay = a.decay[h];
    float step = 1.0f;                              // decay^seg_len, by multiplication in 32-bit
    for (int i = 0; i < a.seg_len; ++i) step *= decay;
    for (size_t e = (size_t)blockIdx.z * 1024 + threadIdx.x;
         e < min(per_head, ((size_t)blockIdx.z + 1) * 1024); e += blockDim.x) {
        const size_t at = (size_t)h * per_head + e;
        float S = carried ? a.state[(size_t)slot * per_state + at] : 0.0f;
        for (int s = 0; s < nseg; ++s) {
            a.seg_start[(size_t)(base + s) * per_state + at] = S;
            if (s + 1 < nseg) S = fmaf(step, S, a.seg_own[(size_t)(base + s) * per_state + at]);
        }
    }
}

// Steps of few tokens: ONE launch instead of three.  A CTA per (head, request) holds all of the
// head's value columns (vdim * lanes threads), rotates q and k of its tokens itself, runs the
// recurrence from and to the slot, and finishes every token in place: unit RMS over the head's
// values, the gate, the activation type.  The sums are those of the three kernels, in their order.
struct StepArgs {
    ScanArgs scan;            // cols == vdim
    const float* freq;
    int rot_dims;
    float k_scale, eps;
    void* out;                // [T, out_ld] in O
    long out_ld;
    int g_col;                // column of the gate in proj, or -1
};

template <int RET_NI, typename O>
__global__ void retention_step_kernel(StepArgs sa) {
    extern __shared__ __align__(16) float smem[];
    __shared__ float inv_s;
    const ScanArgs& a = sa.scan;
    prb_grid_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    if (t1 <= t0 || t0 < 0 || t1 > a.n_tokens) return;
    const int R = a.lanes, dim_pad = R * RET_NI;
    float* qs = smem;                               // [dim_pad]
    float* ks = qs + dim_pad;                       // [dim_pad]
    float* os = ks + dim_pad;                       // [vdim]
    const int r = threadIdx.x % R, col = threadIdx.x / R;
    const bool live = col < a.vdim;
    const int slot = a.state_slot[b];
    if (slot < 0 || slot >= a.n_slots) {
        if (threadIdx.x == 0) prb_set_status(a.status, PRB_S_SLOT_RANGE, t0, slot, a.n_slots);
        return;
    }
    float* srow = a.state + (((size_t)slot * a.heads + h) * a.vdim + (live ? col : 0)) * a.dim;
    const bool carried = a.positions[t0] > 0;
    float S[RET_NI];
#pragma unroll
    for (int ii = 0; ii < RET_NI; ++ii) {
        const int i = r * RET_NI + ii;
        S[ii] = (live && carried && i < a.dim) ? srow[i] : 0.0f;
    }
    const float decay = a.decay[h];
    const int half = sa.rot_dims / 2;
    const int units = half + (a.dim - sa.rot_dims);
    O* out = reinterpret_cast<O*>(sa.out);
    for (int t = t0; t < t1; ++t) {
        __syncthreads();                            // the token before is done with shared memory
        const float* row = a.proj + (size_t)t * a.ld;
        const float* qr = row + a.q_col + h * a.dim;
        const float* kr = row + a.k_col + h * a.dim;
        const float pos = (float)a.positions[t];
        for (int w = threadIdx.x; w < units; w += blockDim.x) {
            if (w < half) {
                float sn, cs;
                sincosf(pos * sa.freq[w], &sn, &cs);
                const float q0 = qr[w], q1 = qr[w + half], k0 = kr[w], k1 = kr[w + half];
                qs[w] = q0 * cs - q1 * sn;
                qs[w + half] = q1 * cs + q0 * sn;
                ks[w] = (k0 * cs - k1 * sn) * sa.k_scale;
                ks[w + half] = (k1 * cs + k0 * sn) * sa.k_scale;
            } else {
                const int i = w - half + sa.rot_dims;
                qs[i] = qr[i];
                ks[i] = kr[i] * sa.k_scale;
            }
        }
        for (int i = a.dim + threadIdx.x; i < dim_pad; i += blockDim.x) qs[i] = ks[i] = 0.0f;
        __syncthreads();
        const float v = live ? row[a.v_col + h * a.vdim + col] : 0.0f;
        const float4* q4 = reinterpret_cast<const float4*>(qs + r * RET_NI);
        const float4* k4 = reinterpret_cast<const float4*>(ks + r * RET_NI);
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int g = 0; g < RET_NI / 4; ++g) {
            const float4 kk = k4[g], qq = q4[g];
            S[4 * g + 0] = fmaf(decay, S[4 * g + 0], kk.x * v);
            S[4 * g + 1] = fmaf(decay, S[4 * g + 1], kk.y * v);
            S[4 * g + 2] = fmaf(decay, S[4 * g + 2], kk.z * v);
            S[4 * g + 3] = fmaf(decay, S[4 * g + 3], kk.w * v);
            acc[0] = fmaf(S[4 * g + 0], qq.x, acc[0]);
            acc[1] = fmaf(S[4 * g + 1], qq.y, acc[1]);
            acc[2] = fmaf(S[4 * g + 2], qq.z, acc[2]);
            acc[3] = fmaf(S[4 * g + 3], qq.w, acc[3]);
        }
        float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        for (int m = 1; m < R; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
        if (live && r == 0) os[col] = o;
        __syncthreads();
        if (threadIdx.x < 32) {                     // the head's unit RMS, as retention_finish sums it
            float ss = 0.0f;
            for (int j = threadIdx.x; j < a.vdim; j += 32) ss = fmaf(os[j], os[j], ss);
            ss = prb_warp_sum(ss);
            if (threadIdx.x == 0) inv_s = 1.0f / sqrtf(ss / (float)a.vdim + sa.eps);
        }
        __syncthreads();
        if (live && r == 0) {
            float y = o * inv_s;
            if (sa.g_col >= 0) {
                const float z = row[sa.g_col + h * a.vdim + col];
                y *= z / (1.0f + expf(-z));
            }
            out[(size_t)t * sa.out_ld + h * a.vdim + col] = prb_from_float<O>(y);
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < RET_NI; ++ii) {
            const int i = r * RET_NI + ii;
            if (i < a.dim) srow[i] = S[ii];
        }
    }
}

template <typename O>
__global__ void retention_finish_kernel(O* __restrict__ out, long out_ld, const float* __restrict__ o_raw,
                                        const float* __restrict__ proj, long ld, int g_col,
                                        const int* __restrict__ seq, int n_tokens, int heads,
                                        int vdim, float eps) {
    prb_grid_launch_dependents();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (unit >= n_tokens * heads) return;
    const int t = unit / heads, h = unit - t * heads;
    O* o = out + (size_t)t * out_ld + h * vdim;
    if (seq[t] < 0) {                               // a padding row
        for (int j = lane; j < vdim; j += 32) o[j] = prb_from_float<O>(0.0f);
        return;
    }
    const float* raw = o_raw + (size_t)t * heads * vdim + h * vdim;
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) ss = fmaf(raw[j], raw[j], ss);
    ss = prb_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const float* g = proj ? proj + (size_t)t * ld + g_col + h * vdim : nullptr;
    for (int j = lane; j < vdim; j += 32) {
        float v = raw[j] * inv;
        if (g) {
            const float z = g[j];
            v *= z / (1.0f + expf(-z));
        }
        o[j] = prb_from_float<O>(v);
    }
}
}  // namespace

// State numbers a lane holds, and lanes a column's dim numbers are spread over (0: a head size
// the scan does not take).
static int ret_ni(int dim) { return dim <= 128 ? 4 : 16; }
PRB_API int prb_retention_lanes(int dim) {
    if (dim <= 0) return 0;
    const int ni = ret_ni(dim);
    int r = 1;
    while (r * ni < dim) r <<= 1;
    return r <= 32 ? r : 0;
}

// Tokens of a segment, and the most segments a step of `t_cap` token rows and `b_cap` requests
// can have (what the two workspaces are sized for).
PRB_API int prb_retention_segment() { return 64; }
PRB_API int prb_retention_max_segments(int t_cap, int b_cap) {
    return t_cap / prb_retention_segment() + b_cap;
}

template <int NI>
static void launch_scan(const ScanArgs& a, int mode, dim3 grid, int threads, size_t smem,
                        cudaStream_t stream) {
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(retention_scan_kernel<NI, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(retention_scan_kernel<NI, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(retention_scan_kernel<NI, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (mode == 0) retention_scan_kernel<NI, 0><<<grid, threads, smem, stream>>>(a);
    else if (mode == 1) retention_scan_kernel<NI, 1><<<grid, threads, smem, stream>>>(a);
    else retention_scan_kernel<NI, 2><<<grid, threads, smem, stream>>>(a);
}

// Rotates q and k IN PLACE in `proj` (and scales k), then runs the scan: by one CTA per
// (columns, head, request), or, with workspaces (`seg_own`, `seg_start`: room for `segments`
// states each), in segments side by side (three launches).
PRB_API int prb_retention_scan(float* o_raw, float* proj, long ld, int q_col, int k_col,
                               int v_col, float* state, const int* q_start, const int* state_slot,
                               const int* positions, const float* decay, const float* freq,
                               int n_tokens, int n_requests, int n_slots, int heads, int dim,
                               int vdim, int rot_dims, float k_scale, int cols, float* seg_own,
                               float* seg_start, int segments, int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    const int lanes = prb_retention_lanes(dim);
    if (heads <= 0 || heads > 65535 || n_requests > 65535 || dim <= 0 || vdim <= 0 || lanes == 0 ||
        rot_dims < 0 || rot_dims > dim || rot_dims % 2 != 0 || cols <= 0)
        return PRB_E_SIZE;
    if (ld % 4 != 0 || ((uintptr_t)proj) % 16 != 0) return PRB_E_ALIGN;
    const bool segmented = seg_own != nullptr && seg_start != nullptr && segments > 0;
    if (segmented && (segments > 65535 || segments < prb_retention_max_segments(n_tokens, n_requests)))
        return PRB_E_SIZE;
    if (rot_dims > 0 || k_scale != 1.0f) {
        const int work = heads * (dim - rot_dims / 2);
        const int rt = work >= 256 ? 256 : ((work + 31) / 32) * 32;
        retention_rotate_kernel<<<n_tokens, rt, 0, stream>>>(proj, ld, q_col, k_col, positions, freq,
                                                             n_tokens, heads, dim, rot_dims, k_scale);
        PRB_LAUNCH_CHECK();
    }
    // threads: cols * lanes rounded up to whole warps, at most 1,024
    if (cols > vdim) cols = vdim;
    while (cols * lanes > 1024) cols = (cols + 1) / 2;
    const int threads = (cols * lanes + 31) / 32 * 32;
    const int chunks = (vdim + cols - 1) / cols;
    const int ni = ret_ni(dim);
    ScanArgs a{o_raw, proj, ld, q_col, k_col, v_col, state, q_start, state_slot, positions, decay,
               n_tokens, n_slots, heads, dim, vdim, cols, lanes, status, n_requests,
               segmented ? prb_retention_segment() : 0, seg_own, seg_start};
    const size_t smem = (size_t)RET_BLOCK * (2 * lanes * ni + cols) * sizeof(float);
    if (!segmented) {
        const dim3 grid(chunks, heads, n_requests);
        if (ni == 4) launch_scan<4>(a, 0, grid, threads, smem, stream);
        else launch_scan<16>(a, 0, grid, threads, smem, stream);
        PRB_LAUNCH_CHECK();
        return 0;
    }
    const dim3 grid(chunks, heads, prb_retention_max_segments(n_tokens, n_requests));
    if (ni == 4) launch_scan<4>(a, 1, grid, threads, smem, stream);
    else launch_scan<16>(a, 1, grid, threads, smem, stream);
    PRB_LAUNCH_CHECK();
    retention_carry_kernel<<<dim3(heads, n_requests, ((size_t)vdim * dim + 1023) / 1024), 256, 0, stream>>>(a);
    PRB_LAUNCH_CHECK();
    if (ni == 4) launch_scan<4>(a, 2, grid, threads, smem, stream);
    else launch_scan<16>(a, 2, grid, threads, smem, stream);
    PRB_LAUNCH_CHECK();
    return 0;
}

PRB_API int prb_retention_finish(void* out, long out_ld, const float* o_raw, const float* proj, long ld,
                                 int g_col, const int* seq, int n_tokens, int heads, int vdim,
                                 float eps, int out_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0) return PRB_E_SIZE;
    const int warps = 4;
    const unsigned blocks = (unsigned)(((size_t)n_tokens * heads + warps - 1) / warps);
    if (out_dtype == PRB_F32)
        retention_finish_kernel<float><<<blocks, warps * 32, 0, stream>>>(
            (float*)out, out_ld, o_raw, proj, ld, g_col, seq, n_tokens, heads, vdim, eps);
    else if (out_dtype == PRB_BF16)
        retention_finish_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
            (__nv_bfloat16*)out, out_ld, o_raw, proj, ld, g_col, seq, n_tokens, heads, vdim, eps);
    else
        return PRB_E_DTYPE;
    PRB_LAUNCH_CHECK();
    return 0;
}

// 1 when the one-launch form takes these sizes (all of a head's columns in one CTA).
PRB_API int prb_retention_step_supports(int dim, int vdim) {
    const int lanes = prb_retention_lanes(dim);
    return lanes > 0 && (long)vdim * lanes <= 1024 ? 1 : 0;
}

// Rotation, recurrence and finish of a step of few tokens in one launch (see
// retention_step_kernel); out in the activation type, its rows out_ld apart.
PRB_API int prb_retention_step(void* out, long out_ld, const float* proj, long ld, int q_col,
                               int k_col, int v_col, int g_col, float* state, const int* q_start,
                               const int* state_slot, const int* positions, const float* decay,
                               const float* freq, int n_tokens, int n_requests, int n_slots,
                               int heads, int dim, int vdim, int rot_dims, float k_scale, float eps,
                               int out_dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    const int lanes = prb_retention_lanes(dim);
    if (heads <= 0 || heads > 65535 || n_requests > 65535 || dim <= 0 || vdim <= 0 ||
        !prb_retention_step_supports(dim, vdim) || rot_dims < 0 || rot_dims > dim || rot_dims % 2 != 0)
        return PRB_E_SIZE;
    if (ld % 4 != 0 || ((uintptr_t)proj) % 16 != 0) return PRB_E_ALIGN;
    const int ni = ret_ni(dim);
    const int threads = (vdim * lanes + 31) / 32 * 32;
    StepArgs sa{ScanArgs{nullptr, proj, ld, q_col, k_col, v_col, state, q_start, state_slot,
                         positions, decay, n_tokens, n_slots, heads, dim, vdim, vdim, lanes, status,
                         n_requests, 0, nullptr, nullptr},
                freq, rot_dims, k_scale, eps, out, out_ld, g_col};
    const size_t smem = (size_t)(2 * lanes * ni + vdim) * sizeof(float);
    const dim3 grid(heads, n_requests);
    if (out_dtype == PRB_F32) {
        if (ni == 4) retention_step_kernel<4, float><<<grid, threads, smem, stream>>>(sa);
        else retention_step_kernel<16, float><<<grid, threads, smem, stream>>>(sa);
    } else if (out_dtype == PRB_BF16) {
        if (ni == 4) retention_step_kernel<4, __nv_bfloat16><<<grid, threads, smem, stream>>>(sa);
        else retention_step_kernel<16, __nv_bfloat16><<<grid, threads, smem, stream>>>(sa);
    } else {
        return PRB_E_DTYPE;
    }
    PRB_LAUNCH_CHECK();
    return 0;
}
