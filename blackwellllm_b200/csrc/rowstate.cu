// Row kernels whose result for a token depends on the token before it, and that therefore carry a little state
// from a request's last token of one step to its first token of the next (the state lives in the cache manager's
// fixed-size slots, one per live request):
//   * embed_bigram: embedding row plus a row of a second table chosen by a hash of (previous token, token);
//   * rmsnorm_shift: RMS norm of the stream, and beside it the same row moved toward the previous token's normed
//     row channel by channel (token shift);
//   * concat2_cast: two float32 streams side by side in the compute type (the operand of a product that mixes them).
// A step's tokens of a request are consecutive rows (cu_q); the first of them reads the state, and the block that
// reads a slot's state is the one that writes its new value afterwards, so no other block touches it.
// All arithmetic is float32.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

// out[t] = table[id] * scale + second[row],  row = (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets`
// (the table's last) for a sequence's first token.  prev_token: int32 [slots], the last token a request has seen.
template <typename WT>
__global__ void embed_bigram_kernel(const WT* __restrict__ table, const WT* __restrict__ second,
                                    const int* __restrict__ ids, const int* __restrict__ positions,
                                    const int* __restrict__ req_of_token, const int* __restrict__ cu_q,
                                    const int* __restrict__ state_slot, int* __restrict__ prev_token,
                                    float* __restrict__ out, int H, int V, int buckets, long long mul_prev,
                                    long long mul_cur, float scale) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    const bool first = t == cu_q[r];
    int id = ids[t];
    if (id < 0 || id >= V) id = 0;  // the host rejects such ids before the launch
    const int pos = positions[t];
    long long row = buckets;
    if (pos > 0) {
        long long prev = first ? prev_token[state_slot[r]] : ids[t - 1];
        row = (prev * mul_prev + (long long)id * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const WT* e = table + (size_t)id * H;
    const WT* b = second + (size_t)row * H;
    float* o = out + (size_t)t * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = bw::to_f32(e[c]) * scale + bw::to_f32(b[c]);
    if (first) {
        __syncthreads();   // every thread has read the old state
        if (threadIdx.x == 0) prev_token[state_slot[r]] = ids[cu_q[r + 1] - 1];
    }
}

// h[t] = x[t] / rms(x[t]) * gain (optional output), hs[t] = h[t] + (h[t-1] - h[t]) * shift, with h[t-1] = 0 at position 0
// and = state[slot] for the first token of a later portion; state[slot] <- h of the request's last token of the step.
// One block per token; the previous row's norm is made again from the stream (it is in L2).
template <typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_shift_kernel(const float* __restrict__ x, const float* __restrict__ gain, const float* __restrict__ shift,
                     float* __restrict__ state, const int* __restrict__ positions, const int* __restrict__ req_of_token,
                     const int* __restrict__ cu_q, const int* __restrict__ state_slot, OT* __restrict__ h_out,
                     OT* __restrict__ hs_out, int H, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int r = req_of_token[t];
    const bool first = t == cu_q[r];
    const int pos = positions[t];
    const float* xr = x + (size_t)t * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
    const float r0 = rsqrtf(bw::block_sum(ss, scratch) / (float)H + eps);
    const float* xp = nullptr;      // the previous token's row of the stream, if it is in this step
    float r1 = 0.f;
    if (pos > 0 && !first) {
        xp = xr - H;
        float sp = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = xp[c]; sp = fmaf(v, v, sp); }
        r1 = rsqrtf(bw::block_sum(sp, scratch) / (float)H + eps);
    }
    float* st = state + (size_t)state_slot[r] * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float g = gain[c];
        const float h = xr[c] * r0 * g;
        float prev = 0.f;
        if (xp) prev = xp[c] * r1 * g;
        else if (pos > 0) prev = st[c];
        if (h_out) h_out[(size_t)t * H + c] = bw::from_f32<OT>(h);
        hs_out[(size_t)t * H + c] = bw::from_f32<OT>(h + (prev - h) * shift[c]);
    }
    if (first) {
        // the new state: the normed row of the request's last token of this step (each thread writes the
        // channels it has read above)
        const int last = cu_q[r + 1] - 1;
        const float* xl = x + (size_t)last * H;
        float rl = r0;
        if (last != t) {
            float sl = 0.f;
            for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = xl[c]; sl = fmaf(v, v, sl); }
            rl = rsqrtf(bw::block_sum(sl, scratch) / (float)H + eps);
        }
        for (int c = threadIdx.x; c < H; c += blockDim.x) st[c] = xl[c] * rl * gain[c];
    }
}

template <typename OT>
__global__ void concat2_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, OT* __restrict__ out, int H) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        out[t * 2 * H + c] = bw::from_f32<OT>(a[t * H + c]);
        out[t * 2 * H + H + c] = bw::from_f32<OT>(b[t * H + c]);
    }
}

}  // namespace

// table [V, H] and second [buckets + 1, H] of the same type; out float32 [T, H]; prev_token int32 [slots].
BW_EXPORT int bw_embed_bigram(const void* table, const void* second, int table_type, const int* ids, const int* positions,
                              const int* req_of_token, const int* cu_q, const int* state_slot, int* prev_token, float* out,
                              int T, int H, int V, int buckets, long long mul_prev, long long mul_cur, float scale, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0 || buckets <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 256 ? 256 : 128;
    if (table_type == BW_F32)
        bw::launch((embed_bigram_kernel<float>), dim3(T), dim3(threads), 0, s, (const float*)table, (const float*)second, ids,
                   positions, req_of_token, cu_q, state_slot, prev_token, out, H, V, buckets, mul_prev, mul_cur, scale);
    else if (table_type == BW_BF16)
        bw::launch((embed_bigram_kernel<bf16>), dim3(T), dim3(threads), 0, s, (const bf16*)table, (const bf16*)second, ids,
                   positions, req_of_token, cu_q, state_slot, prev_token, out, H, V, buckets, mul_prev, mul_cur, scale);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// x float32 [T, H]; gain, shift float32 [H]; state float32 [slots, H]; h_out (may be null) and hs_out [T, H] of out_type.
BW_EXPORT int bw_rmsnorm_shift(const float* x, const float* gain, const float* shift, float* state, const int* positions,
                               const int* req_of_token, const int* cu_q, const int* state_slot, void* h_out, void* hs_out,
                               int out_type, int T, int H, float eps, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || !hs_out) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32)
        bw::launch((rmsnorm_shift_kernel<float>), dim3(T), dim3(256), 0, s, x, gain, shift, state, positions, req_of_token,
                   cu_q, state_slot, (float*)h_out, (float*)hs_out, H, eps);
    else if (out_type == BW_BF16)
        bw::launch((rmsnorm_shift_kernel<bf16>), dim3(T), dim3(256), 0, s, x, gain, shift, state, positions, req_of_token,
                   cu_q, state_slot, (bf16*)h_out, (bf16*)hs_out, H, eps);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// out [T, 2H] of out_type = (a | b), both float32 [T, H].
BW_EXPORT int bw_concat2_cast(const float* a, const float* b, void* out, int out_type, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32) bw::launch((concat2_cast_kernel<float>), dim3(T), dim3(256), 0, s, a, b, (float*)out, H);
    else if (out_type == BW_BF16) bw::launch((concat2_cast_kernel<bf16>), dim3(T), dim3(256), 0, s, a, b, (bf16*)out, H);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
