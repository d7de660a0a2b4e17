// Matrix memory with exponential gates (mLSTM): the parts around the recurrence itself, which is the scan of gla.cu
// (one decay per head and token, keys times the input gate, a column of ones that carries the normaliser).
//
//   i_t = cap tanh((w_i . x_t + b_i) / cap)                     log input gate, per head
//   f_t = log_sigmoid(cap tanh((w_f . x_t + b_f) / cap))        log forget gate, per head
//   m_t = max(f_t + m_(t-1), i_t)                               m starts at 0
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        n_t likewise with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//   y_t = o_t / rms(o_t) * gain * sigmoid(g_t)                  rms per head, gain per channel of all heads
//
// mlstm_gates_kernel makes a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t) and e_t = exp(-m_t) for a step's tokens,
// request by request in order, from and into the request's m; mlstm_out_kernel makes y from the scan's output, whose
// last column per head is n_t . q_t.  Everything here is float32.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// One block per (request, head).  First all its warps make the two gates of the segment's tokens (the transcendental
// part, a token a thread) and park them in the a and b outputs; then warp 0 walks the segment in stretches of 32 tokens:
// the stretch's gates go to shared memory, the chain m_t = max(f_t + m_(t-1), i_t) runs through them in order on every
// lane (an addition and a maximum a token, the gates read as broadcasts that do not wait for the chain), each lane keeping
// the m before and after its own token, then the lane's three exponentials.  The chain's order is the tokens' order, so
// the result does not depend on how the tokens were cut into steps.
constexpr int GATE_THREADS = 256;
__global__ void __launch_bounds__(GATE_THREADS)
mlstm_gates_kernel(const float* __restrict__ proj, long long ld, int i_off, int f_off, const float* __restrict__ bias_i,
                   const float* __restrict__ bias_f, float cap, const int* __restrict__ cu_q,
                   const int* __restrict__ state_slot, float* __restrict__ m_state, float* a_out, float* b_out,
                   float* __restrict__ e_out, int R, int heads) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float2 gates[32];     // (f, i) of the stretch's tokens
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x / heads, h = blockIdx.x - r * heads;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    if (t0 >= t1) return;
    const float bi = bias_i[h], bf = bias_f[h], inv_cap = 1.f / cap;
    for (int t = t0 + threadIdx.x; t < t1; t += GATE_THREADS) {
        const float* row = proj + (size_t)t * ld;
        const size_t o = (size_t)t * heads + h;
        b_out[o] = cap * tanhf((row[i_off + h] + bi) * inv_cap);
        a_out[o] = log_sigmoid(cap * tanhf((row[f_off + h] + bf) * inv_cap));
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    float* mp = m_state + (size_t)state_slot[r] * heads + h;
    float m = *mp;
    float gi = 0.f, gf = 0.f;
    if (t0 + lane < t1) { const size_t o = (size_t)(t0 + lane) * heads + h; gf = a_out[o]; gi = b_out[o]; }
    for (int tb = t0; tb < t1; tb += 32) {
        const int t = tb + lane;
        const float my_f = gf, my_i = gi;
        __syncwarp();
        gates[lane] = make_float2(gf, gi);
        __syncwarp();
        if (t + 32 < t1) { const size_t o = (size_t)(t + 32) * heads + h; gf = a_out[o]; gi = b_out[o]; }   // the next stretch travels
        const int n = min(32, t1 - tb);
        float m_before = 0.f, m_after = 0.f;
        if (n == 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float2 g = gates[j];
                const float m_new = fmaxf(g.x + m, g.y);
                if (j == lane) { m_before = m; m_after = m_new; }
                m = m_new;
            }
        } else {
            for (int j = 0; j < n; ++j) {
                const float2 g = gates[j];
                const float m_new = fmaxf(g.x + m, g.y);
                if (j == lane) { m_before = m; m_after = m_new; }
                m = m_new;
            }
        }
        if (t < t1) {
            const size_t o = (size_t)t * heads + h;
            a_out[o] = expf(my_f + m_before - m_after);
            b_out[o] = expf(my_i - m_after);
            e_out[o] = expf(-m_after);
        }
    }
    if (lane == 0) *mp = m;
}

// One warp per (token, head): the scan's output o [T, heads * (dv + 1)], the head's last column being n . q.
template <typename OT>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ e, const float* __restrict__ g, long long g_ld,
                 int g_off, const float* __restrict__ gain, OT* __restrict__ out, int T, int heads, int dv, float eps,
                 float den_eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const int t = item / heads, h = item - t * heads;
    const float* orow = o + ((size_t)t * heads + h) * (dv + 1);
    const float inv = 1.f / (fmaxf(fabsf(orow[dv]), e[(size_t)t * heads + h]) + den_eps);
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float v = orow[c] * inv; ss = fmaf(v, v, ss); }
    const float r = rsqrtf(bw::warp_sum(ss) / (float)dv + eps);
    const float* grow = g + (size_t)t * g_ld + g_off + (size_t)h * dv;
    OT* dst = out + ((size_t)t * heads + h) * dv;
    for (int c = lane; c < dv; c += 32)
        dst[c] = bw::from_f32<OT>(orow[c] * inv * r * gain[(size_t)h * dv + c] / (1.f + expf(-grow[c])));
}

}  // namespace

// proj: float32 [T, ld], the gates' projections at columns i_off and f_off (heads columns each); bias_i, bias_f: float32
// [heads]; m_state: float32 [slots, heads]; a, b, e: float32 [T, heads] out.
BW_EXPORT int bw_mlstm_gates(const float* proj, long long ld, int i_off, int f_off, const float* bias_i, const float* bias_f,
                             float cap, const int* cu_q, const int* state_slot, float* m_state, float* a, float* b, float* e,
                             int R, int heads, void* stream) {
    if (R <= 0) return 0;
    if (heads <= 0 || !(cap > 0.f) || !bias_i || !bias_f || ld < (long long)i_off + heads || ld < (long long)f_off + heads)
        return BW_ERR_BAD_ARG;
    bw::launch(mlstm_gates_kernel, dim3(R * heads), dim3(GATE_THREADS), 0, (cudaStream_t)stream, proj, ld, i_off, f_off, bias_i,
               bias_f, cap, cu_q, state_slot, m_state, a, b, e, R, heads);
    BW_LAUNCH_CHECK();
    return 0;
}

// o: float32 [T, heads * (dv + 1)] (the scan's output); e: float32 [T, heads]; g: float32 rows g_ld apart, the output gate's
// projection at column g_off (heads * dv columns); gain: float32 [heads * dv]; out: [T, heads * dv] of out_type.
BW_EXPORT int bw_mlstm_out(const float* o, const float* e, const float* g, long long g_ld, int g_off, const float* gain,
                           void* out, int out_type, int T, int heads, int dv, float eps, float den_eps, void* stream) {
    if (T <= 0) return 0;
    if (heads <= 0 || dv <= 0 || g_ld < (long long)g_off + (long long)heads * dv) return BW_ERR_BAD_ARG;
    const dim3 grid((T * heads + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32) bw::launch((mlstm_out_kernel<float>), grid, dim3(128), 0, s, o, e, g, g_ld, g_off, gain, (float*)out, T, heads, dv, eps, den_eps);
    else if (out_type == BW_BF16) bw::launch((mlstm_out_kernel<bf16>), grid, dim3(128), 0, s, o, e, g, g_ld, g_off, gain, (bf16*)out, T, heads, dv, eps, den_eps);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
