// Gated linear attention: a recurrent mixer with a matrix state per head and a decay per key channel.
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dk, dv] per head, float32, one per request
//   o_t = S_t^T q_t                            q scaled by q_scale
//   a_t = sigmoid(z_t) ^ (1 / tau) = exp(log_sigmoid(z_t) / tau),   z_t = W2 (W1 x_t) + b
//
// Everything but the projections that make q, k, v, z is float32 here: the decay and its logarithm,
// the state, the products that enter and leave it, and the norm of the head's output.
//
// gla_scan_kernel walks the tokens of one request's segment in order (a single decoded token and a
// portion of a prompt are the same case), from the state the steps before left in the request's slot,
// and leaves the new state there.  A block owns (request, head, COLS value columns); a warp owns CPT of
// them, their dk state rows spread over its lanes, in registers.  The order of all sums
// depends on dk alone, never on how the tokens were cut into steps or on the batch.  The scan is a chain
// through the tokens (state in float32, as the design asks): it is bound by the latency of one token's
// update, not by memory or arithmetic throughput, and its parallelism is requests x heads x columns / COLS.
//
// gla_decay_kernel makes a_t from the first projection's result (W2 has a small inner size: float32 FMAs).
// gla_gate_kernel: per token and head, o / rms(o) * gain * silu(g) -> the output projection's operand.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int COLS = 32;        // value columns of a block
constexpr int CPT = 4;          // value columns of a warp (and of each of its lanes)
constexpr int THREADS = 32 * COLS / CPT;
constexpr int MAX_DK = 256;
constexpr int TOK_CHUNK = 16;   // tokens staged in shared memory at a time

struct ScanParams {
    const float* qkv;      // [T, ld]: q at q_off, k at k_off, v at v_off (head-major within each)
    const float* decay;    // [T, heads * dk]: a_t, already in (0, 1)
    const int* cu_q;       // [R + 1]
    const int* state_slot; // [R]
    float* state;          // [slots, heads, dk, dv]
    float* o;              // [T, heads * dv]
    long long ld;
    int q_off, k_off, v_off;
    int heads, dk, dv;
    float q_scale;
    // The same recurrence serves a matrix memory with ONE decay per head and token and a normaliser:
    // scalar_decay != 0: decay is [T, heads] (a_t of the head, used for every key channel);
    // k_scale != null: [T, heads], the token's keys are multiplied by it as they are read (an input gate);
    // ones_col != 0: the head's last value column (dv - 1) is the constant 1 and v holds dv - 1 columns a head, so that
    // column of the state is n_t = a_t n_(t-1) + k_t and the last output column is n_t . q_t.
    const float* k_scale;
    int scalar_decay, ones_col;
    int sld;               // floats between the state's rows (>= dv; columns from dv on stay zero)
};

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(1 / (1 + exp(-z))) without overflow on either side
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// a[t, c] = sigmoid(z)^(1 / tau) with z = sum_r x[t, r] w[c, r] + b[c]: the decay's second projection (its inner
// size is small), the sigmoid's logarithm, the division by tau and the exponential, all float32.
// x: float32 [T, ldx] at column x_off; w: [C, rank] (float32 or bfloat16); one thread per (t, c).
template <typename WT>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ x, long long ldx, int x_off, const WT* __restrict__ w,
                 const WT* __restrict__ b, float* __restrict__ a, int T, int C, int rank, float inv_tau) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T * C) return;
    const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
    const float* xr = x + (size_t)t * ldx + x_off;
    const WT* wr = w + (size_t)c * rank;
    float z = 0.f;
    for (int r = 0; r < rank; ++r) z = fmaf(xr[r], bw::to_f32(wr[r]), z);
    z += bw::to_f32(b[c]);
    a[idx] = expf(log_sigmoid(z) * inv_tau);
}

// RPL: state rows per lane (a multiple of 4): dk <= 32 * RPL.  A warp owns CPT value columns and all key
// channels: lane l holds channels (j * 32 + l) * 4 + e (j < RPL / 4, e < 4) of each of its columns, so a token's
// q, k and a values are read from shared memory once per warp (16-byte loads, 512 consecutive bytes a warp)
// and used for CPT columns.  In shared memory a token's rows are padded with zeros to DKP = 32 * RPL channels
// (a padded channel stays at zero and adds nothing), so the inner loop has no bounds.  The CPT sums over the
// 32 lanes take six shuffles: two that halve the number of columns a lane carries, then three over what is left.
// MEM: the form for a matrix memory (ScanParams: one decay per head, keys times k_scale, the column of ones); the plain
// form's code does not know of it.  What a fetch loads is not touched before it is staged: a thread never waits for a
// load inside the fetch, so the key's scale travels in registers of its own and multiplies at staging.
template <int RPL, bool MEM>
__global__ void __launch_bounds__(THREADS)
gla_scan_kernel(ScanParams p) {
    BW_PDL_TRIGGER();
    constexpr int DKP = 32 * RPL;
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;                          // [TOK_CHUNK][DKP]
    float* ks = qs + TOK_CHUNK * DKP;
    float* as = ks + TOK_CHUNK * DKP;
    float* vs = as + TOK_CHUNK * DKP;        // [TOK_CHUNK][COLS]
    constexpr int NST = TOK_CHUNK * DKP / THREADS;   // staged values of q, k, a per thread
    constexpr int NSV = TOK_CHUNK * COLS / THREADS;
    const int r = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cbase = c0 + warp * CPT;
    const int t0 = p.cu_q[r], t1 = p.cu_q[r + 1];
    float* S = p.state + (((size_t)p.state_slot[r] * p.heads + h) * p.dk) * p.sld;
    BW_PDL_WAIT();
    float s[RPL][CPT];
    const bool vec_state = (p.sld & 3) == 0 && cbase + CPT <= p.sld;   // a lane's CPT columns of a row as one 16-byte access
#pragma unroll
    for (int j = 0; j < RPL; ++j) {
        const int i = ((j >> 2) * 32 + lane) * 4 + (j & 3);
        if (vec_state) {
            const float4 v = i < p.dk ? *reinterpret_cast<const float4*>(S + (size_t)i * p.sld + cbase) : make_float4(0.f, 0.f, 0.f, 0.f);
            s[j][0] = v.x; s[j][1] = v.y; s[j][2] = v.z; s[j][3] = v.w;
        } else {
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) s[j][cc] = (i < p.dk && cbase + cc < p.dv) ? S[(size_t)i * p.sld + cbase + cc] : 0.f;
        }
    }
    // The next chunk's values travel from memory into registers while this chunk is worked on from shared
    // memory, so that their latency is not added to the chain through the tokens.
    float rq[NST], rk[NST], ra[NST], rv[NSV];
    float rs[MEM ? NST : 1];
    const int dv_in = p.dv - ((MEM && p.ones_col) ? 1 : 0);   // value columns a head has in memory
    auto fetch = [&](int tb, int n) {
#pragma unroll
        for (int u = 0; u < NST; ++u) {
            const int idx = threadIdx.x + u * THREADS;
            const int tt = idx / DKP, i = idx % DKP;
            rq[u] = rk[u] = ra[u] = 0.f;
            if constexpr (MEM) rs[u] = 1.f;
            if (tt < n && i < p.dk) {
                const float* row = p.qkv + (size_t)(tb + tt) * p.ld;
                rq[u] = row[p.q_off + h * p.dk + i];
                rk[u] = row[p.k_off + h * p.dk + i];
                if constexpr (MEM) {
                    if (p.k_scale) rs[u] = p.k_scale[(size_t)(tb + tt) * p.heads + h];
                    ra[u] = p.scalar_decay ? p.decay[(size_t)(tb + tt) * p.heads + h]
                                           : p.decay[(size_t)(tb + tt) * p.heads * p.dk + h * p.dk + i];
                } else {
                    ra[u] = p.decay[(size_t)(tb + tt) * p.heads * p.dk + h * p.dk + i];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < NSV; ++u) {
            const int idx = threadIdx.x + u * THREADS;
            const int tt = idx / COLS, cc = idx % COLS;
            rv[u] = (tt < n && c0 + cc < dv_in) ? p.qkv[(size_t)(tb + tt) * p.ld + p.v_off + h * dv_in + c0 + cc]
                                                : ((MEM && tt < n && p.ones_col && c0 + cc == dv_in) ? 1.f : 0.f);
        }
    };
    if (t0 < t1) fetch(t0, min(TOK_CHUNK, t1 - t0));
    const float4* q4 = reinterpret_cast<const float4*>(qs);
    const float4* k4 = reinterpret_cast<const float4*>(ks);
    const float4* a4 = reinterpret_cast<const float4*>(as);
    const float4* v4 = reinterpret_cast<const float4*>(vs);
    const bool hi16 = lane & 16, hi8 = lane & 8;
    const int my_col = cbase + (hi16 ? 2 : 0) + (hi8 ? 1 : 0);   // the column whose sum ends in this lane (lanes 0, 8, 16, 24)
    for (int tb = t0; tb < t1; tb += TOK_CHUNK) {
        const int n = min(TOK_CHUNK, t1 - tb);
        __syncthreads();                      // the chunk before has been read
#pragma unroll
        for (int u = 0; u < NST; ++u) {
            const int idx = threadIdx.x + u * THREADS;
            qs[idx] = rq[u] * p.q_scale; as[idx] = ra[u];
            if constexpr (MEM) ks[idx] = rk[u] * rs[u]; else ks[idx] = rk[u];
        }
#pragma unroll
        for (int u = 0; u < NSV; ++u) vs[threadIdx.x + u * THREADS] = rv[u];
        __syncthreads();
        if (tb + TOK_CHUNK < t1) fetch(tb + TOK_CHUNK, min(TOK_CHUNK, t1 - tb - TOK_CHUNK));
#pragma unroll 2
        for (int tt = 0; tt < n; ++tt) {
            const float4 vv = v4[tt * (COLS / 4) + warp];
            const float v[CPT] = {vv.x, vv.y, vv.z, vv.w};
            const int base = tt * (DKP / 4) + lane;
            float acc[CPT] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < RPL / 4; ++j) {
                const float4 a = a4[base + j * 32], k = k4[base + j * 32], q = q4[base + j * 32];
                const float ae[4] = {a.x, a.y, a.z, a.w}, ke[4] = {k.x, k.y, k.z, k.w}, qe[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int cc = 0; cc < CPT; ++cc) {
                        s[4 * j + e][cc] = fmaf(ae[e], s[4 * j + e][cc], ke[e] * v[cc]);
                        acc[cc] = fmaf(s[4 * j + e][cc], qe[e], acc[cc]);
                    }
            }
            // lanes 0..15 go on with columns 0 and 1, lanes 16..31 with 2 and 3; then by bit 3 one column each
            const float g0 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[0] : acc[2], 16);
            const float g1 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[1] : acc[3], 16);
            const float b0 = (hi16 ? acc[2] : acc[0]) + g0, b1 = (hi16 ? acc[3] : acc[1]) + g1;
            float sum = (hi8 ? b1 : b0) + __shfl_xor_sync(0xffffffffu, hi8 ? b0 : b1, 8);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if ((lane & 7) == 0 && my_col < p.dv) p.o[(size_t)(tb + tt) * p.heads * p.dv + h * p.dv + my_col] = sum;
        }
    }
#pragma unroll
    for (int j = 0; j < RPL; ++j) {
        const int i = ((j >> 2) * 32 + lane) * 4 + (j & 3);
        if (vec_state) {
            if (i < p.dk) *reinterpret_cast<float4*>(S + (size_t)i * p.sld + cbase) = make_float4(s[j][0], s[j][1], s[j][2], s[j][3]);
        } else {
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc)
                if (i < p.dk && cbase + cc < p.dv) S[(size_t)i * p.sld + cbase + cc] = s[j][cc];
        }
    }
}

// one warp per (token, head): o / sqrt(mean(o^2) + eps) * gain[c] * silu(g[c])
template <typename OT>
__global__ void __launch_bounds__(128)
gla_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, long long g_ld, int g_off,
                const float* __restrict__ gain, OT* __restrict__ out, int T, int heads, int dv, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const int t = item / heads, h = item - t * heads;
    const float* orow = o + (size_t)t * heads * dv + (size_t)h * dv;
    const float* grow = g + (size_t)t * g_ld + g_off + (size_t)h * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = orow[c]; ss = fmaf(v, v, ss); }
    ss = bw::warp_sum(ss);
    const float r = rsqrtf(ss / (float)dv + eps);
    OT* dst = out + (size_t)t * heads * dv + (size_t)h * dv;
    for (int c = lane; c < dv; c += 32) {
        const float gv = grow[c];
        const float sg = gv / (1.f + expf(-gv));
        dst[c] = bw::from_f32<OT>(orow[c] * r * gain[c] * sg);
    }
}

}  // namespace

// decay: float32 [T, heads * dk] from bw_gla_decay; with scalar_decay [T, heads].  k_scale: float32 [T, heads] or null.
// ones_col != 0: dv counts a last column of ones that v does not hold (state [slots, heads, dk, state_ld], o [T, heads * dv]).
// state_ld: floats between the state's rows (0: dv); with a multiple of 4 a lane moves its columns of a row in one access.
BW_EXPORT int bw_gla_scan(const float* qkv, long long ld, int q_off, int k_off, int v_off, const float* decay,
                          const int* cu_q, const int* state_slot, float* state, float* o, int R, int heads, int dk,
                          int dv, float q_scale, const float* k_scale, int scalar_decay, int ones_col, int state_ld,
                          void* stream) {
    if (R <= 0) return 0;
    if (heads <= 0 || dk <= 0 || dv <= 0 || (ones_col && dv < 2) || (state_ld != 0 && state_ld < dv)) return BW_ERR_BAD_ARG;
    if (dk > MAX_DK) return BW_ERR_UNSUPPORTED;
    ScanParams p;
    p.qkv = qkv; p.decay = decay; p.cu_q = cu_q; p.state_slot = state_slot; p.state = state; p.o = o; p.ld = ld;
    p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.heads = heads; p.dk = dk; p.dv = dv;
    p.q_scale = q_scale;
    p.k_scale = k_scale; p.scalar_decay = scalar_decay; p.ones_col = ones_col; p.sld = state_ld ? state_ld : dv;
    const dim3 grid(R, heads, (dv + COLS - 1) / COLS);
    const int rpl = dk <= 128 ? 4 : 8;
    const size_t smem = (size_t)(3 * TOK_CHUNK * 32 * rpl + TOK_CHUNK * COLS) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    const bool mem = k_scale || scalar_decay || ones_col;
    if (rpl == 4) {
        if (mem) bw::launch((gla_scan_kernel<4, true>), grid, dim3(THREADS), smem, s, p);
        else bw::launch((gla_scan_kernel<4, false>), grid, dim3(THREADS), smem, s, p);
    } else {
        static bool raised[bw::MAX_DEVICES] = {}, raised_mem[bw::MAX_DEVICES] = {};
        if (mem) {
            if (bw::allow_dynamic_smem(gla_scan_kernel<8, true>, (int)smem, raised_mem) != cudaSuccess) return BW_ERR_DRIVER;
            bw::launch((gla_scan_kernel<8, true>), grid, dim3(THREADS), smem, s, p);
        } else {
            if (bw::allow_dynamic_smem(gla_scan_kernel<8, false>, (int)smem, raised) != cudaSuccess) return BW_ERR_DRIVER;
            bw::launch((gla_scan_kernel<8, false>), grid, dim3(THREADS), smem, s, p);
        }
    }
    BW_LAUNCH_CHECK();
    return 0;
}

// x: float32 [T, ldx], the decay's first projection at column x_off; w [C, rank] and b [C] of w_type.
BW_EXPORT int bw_gla_decay(const float* x, long long ldx, int x_off, const void* w, const void* b, int w_type, float* a,
                           int T, int C, int rank, float tau, void* stream) {
    if (T <= 0) return 0;
    if (C <= 0 || rank <= 0 || !(tau > 0.f)) return BW_ERR_BAD_ARG;
    const long long total = (long long)T * C;
    const dim3 grid((unsigned)((total + 255) / 256));
    cudaStream_t s = (cudaStream_t)stream;
    if (w_type == BW_F32) bw::launch((gla_decay_kernel<float>), grid, dim3(256), 0, s, x, ldx, x_off, (const float*)w, (const float*)b, a, T, C, rank, 1.f / tau);
    else if (w_type == BW_BF16) bw::launch((gla_decay_kernel<bf16>), grid, dim3(256), 0, s, x, ldx, x_off, (const bf16*)w, (const bf16*)b, a, T, C, rank, 1.f / tau);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_gla_gate(const float* o, const float* g, long long g_ld, int g_off, const float* gain, void* out,
                          int out_type, int T, int heads, int dv, float eps, void* stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || dv <= 0) return BW_ERR_BAD_ARG;
    const int items = T * heads;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32)
        bw::launch((gla_gate_kernel<float>), dim3((items + 3) / 4), dim3(128), 0, s, o, g, g_ld, g_off, gain, (float*)out, T, heads, dv, eps);
    else if (out_type == BW_BF16)
        bw::launch((gla_gate_kernel<bf16>), dim3((items + 3) / 4), dim3(128), 0, s, o, g, g_ld, g_off, gain, (bf16*)out, T, heads, dv, eps);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
