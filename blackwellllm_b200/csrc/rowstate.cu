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

// W consecutive elements (W = 4: one 16-byte access of float32, one 8-byte access of bfloat16; W = 1 for widths
// that are no multiple of 4 or rows that do not start on 16 bytes).  The arithmetic is the same either way.
template <int W> __device__ __forceinline__ void ld(const float* p, float (&v)[W]) {
    if constexpr (W == 4) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    else v[0] = *p;
}
template <int W> __device__ __forceinline__ void ld(const bf16* p, float (&v)[W]) {
    if constexpr (W == 4) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    } else v[0] = __bfloat162float(*p);
}
template <int W> __device__ __forceinline__ void st(float* p, const float (&v)[W]) {
    if constexpr (W == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else *p = v[0];
}
template <int W> __device__ __forceinline__ void st(bf16* p, const float (&v)[W]) {
    if constexpr (W == 4) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t*>(&a); r.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    } else *p = __float2bfloat16(v[0]);
}

// out[t] = table[id] * scale + second[row],  row = (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets`
// (the table's last) for a sequence's first token.  prev_token: int32 [slots], the last token a request has seen.
template <typename WT, int W>
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
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        float ev[W], bv[W];
        ld<W>(e + c, ev); ld<W>(b + c, bv);
#pragma unroll
        for (int j = 0; j < W; ++j) ev[j] = ev[j] * scale + bv[j];
        st<W>(o + c, ev);
    }
    if (first) {
        __syncthreads();   // every thread has read the old state
        if (threadIdx.x == 0) prev_token[state_slot[r]] = ids[cu_q[r + 1] - 1];
    }
}

template <int W> __device__ __forceinline__ float sum_squares(const float* __restrict__ row, int H) {
    float ss = 0.f;
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        float v[W];
        ld<W>(row + c, v);
#pragma unroll
        for (int j = 0; j < W; ++j) ss = fmaf(v[j], v[j], ss);
    }
    return ss;
}

// h[t] = x[t] / rms(x[t]) * gain (optional output), hs[t] = h[t] + (h[t-1] - h[t]) * shift, with h[t-1] = 0 at position 0
// and = state[slot] for the first token of a later portion; state[slot] <- h of the request's last token of the step.
// One block per token; the previous row's norm is made again from the stream (it is in L2).
// planes != null (only in a step whose every request brings ONE token, so that no block reads another block's row):
// a matrix product that its kernel left unsummed; x[t] += planes[0][t] + planes[1][t] + ... first, written back.  Every
// thread re-reads only what it wrote itself.
template <typename OT, int W>
__global__ void __launch_bounds__(1024)
rmsnorm_shift_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes, size_t plane_stride,
                     const float* __restrict__ gain, const float* __restrict__ shift,
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
    float* xr = x + (size_t)t * H;
    float ss = 0.f;
    if (planes) {
        const float* pr = planes + (size_t)t * H;
        for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
            float v[W];
            ld<W>(xr + c, v);
            for (int p0 = 0; p0 < n_planes; p0 += 8) {   // in plane order, eight loads in flight at a time
                float a[8][W];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (p0 + k < n_planes) ld<W>(pr + (size_t)(p0 + k) * plane_stride + c, a[k]);
                    else {
#pragma unroll
                        for (int j = 0; j < W; ++j) a[k][j] = 0.f;
                    }
                }
#pragma unroll
                for (int k = 0; k < 8; ++k)
#pragma unroll
                    for (int j = 0; j < W; ++j) v[j] += a[k][j];
            }
            st<W>(xr + c, v);
#pragma unroll
            for (int j = 0; j < W; ++j) ss = fmaf(v[j], v[j], ss);
        }
    } else {
        ss = sum_squares<W>(xr, H);
    }
    const float r0 = rsqrtf(bw::block_sum(ss, scratch) / (float)H + eps);
    const float* xp = nullptr;      // the previous token's row of the stream, if it is in this step
    float r1 = 0.f;
    if (pos > 0 && !first) {
        xp = xr - H;
        r1 = rsqrtf(bw::block_sum(sum_squares<W>(xp, H), scratch) / (float)H + eps);
    }
    float* stt = state + (size_t)state_slot[r] * H;
    const bool last_here = first && cu_q[r + 1] - 1 == t;   // this row is also the request's last of the step: the new state
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        float xv[W], g[W], sh[W], prev[W], h[W], hs[W];
        ld<W>(xr + c, xv); ld<W>(gain + c, g); ld<W>(shift + c, sh);
        if (xp) {
            ld<W>(xp + c, prev);
#pragma unroll
            for (int j = 0; j < W; ++j) prev[j] = prev[j] * r1 * g[j];
        } else if (pos > 0) {
            ld<W>(stt + c, prev);
        } else {
#pragma unroll
            for (int j = 0; j < W; ++j) prev[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < W; ++j) { h[j] = xv[j] * r0 * g[j]; hs[j] = h[j] + (prev[j] - h[j]) * sh[j]; }
        if (h_out) st<W>(h_out + (size_t)t * H + c, h);
        st<W>(hs_out + (size_t)t * H + c, hs);
        if (last_here) st<W>(stt + c, h);   // (each thread writes the channels it has read above)
    }
    if (first && !last_here) {
        // the new state: the normed row of the request's last token of this step (each thread writes the
        // channels it has read above)
        const float* xl = x + (size_t)(cu_q[r + 1] - 1) * H;
        const float rl = rsqrtf(bw::block_sum(sum_squares<W>(xl, H), scratch) / (float)H + eps);
        for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
            float v[W], g[W];
            ld<W>(xl + c, v); ld<W>(gain + c, g);
#pragma unroll
            for (int j = 0; j < W; ++j) v[j] = v[j] * rl * g[j];
            st<W>(stt + c, v);
        }
    }
}

template <typename OT, int W>
__global__ void concat2_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, OT* __restrict__ out, int H) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        float av[W], bv[W];
        ld<W>(a + t * H + c, av); ld<W>(b + t * H + c, bv);
        st<W>(out + t * 2 * H + c, av);
        st<W>(out + t * 2 * H + H + c, bv);
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// table [V, H] and second [buckets + 1, H] of the same type; out float32 [T, H]; prev_token int32 [slots].
BW_EXPORT int bw_embed_bigram(const void* table, const void* second, int table_type, const int* ids, const int* positions,
                              const int* req_of_token, const int* cu_q, const int* state_slot, int* prev_token, float* out,
                              int T, int H, int V, int buckets, long long mul_prev, long long mul_cur, float scale, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0 || buckets <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    const bool vec = H % 4 == 0 && aligned16(table) && aligned16(second) && aligned16(out);
#define BW_EMB(WT, W) bw::launch((embed_bigram_kernel<WT, W>), dim3(T), dim3(threads), 0, s, (const WT*)table, (const WT*)second, ids, \
                                 positions, req_of_token, cu_q, state_slot, prev_token, out, H, V, buckets, mul_prev, mul_cur, scale)
    if (table_type == BW_F32) { if (vec) BW_EMB(float, 4); else BW_EMB(float, 1); }
    else if (table_type == BW_BF16) { if (vec) BW_EMB(bf16, 4); else BW_EMB(bf16, 1); }
    else return BW_ERR_BAD_ARG;
#undef BW_EMB
    BW_LAUNCH_CHECK();
    return 0;
}

// x float32 [T, H]; gain, shift float32 [H]; state float32 [slots, H]; h_out (may be null) and hs_out [T, H] of out_type.
// planes (may be null): n_planes float32 [T, H] planes, plane_stride floats apart, that are added into x first; only
// for a step whose every request brings one token (the caller's promise: rows are then independent of one another).
BW_EXPORT int bw_rmsnorm_shift(float* x, const float* planes, int n_planes, long long plane_stride, const float* gain,
                               const float* shift, float* state, const int* positions,
                               const int* req_of_token, const int* cu_q, const int* state_slot, void* h_out, void* hs_out,
                               int out_type, int T, int H, float eps, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || !hs_out || (planes && (n_planes <= 0 || plane_stride < (long long)T * H))) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && aligned16(x) && aligned16(gain) && aligned16(shift) && aligned16(state) && aligned16(hs_out) &&
                     aligned16(h_out) && (!planes || (aligned16(planes) && plane_stride % 4 == 0));
    // with planes (a few rows): a thread per four elements, up to 1,024, so that the loads of the stream and of the
    // planes are in flight at once
    int threads = H >= 1024 ? 256 : 128;
    if (planes) { const int quads = (H / (vec ? 4 : 1) + 31) / 32 * 32; threads = quads > 1024 ? 1024 : (quads < 128 ? 128 : quads); }
#define BW_RS(OT, W) bw::launch((rmsnorm_shift_kernel<OT, W>), dim3(T), dim3(threads), 0, s, x, planes, n_planes, (size_t)plane_stride, \
                                gain, shift, state, positions, req_of_token, cu_q, state_slot, (OT*)h_out, (OT*)hs_out, H, eps)
    if (out_type == BW_F32) { if (vec) BW_RS(float, 4); else BW_RS(float, 1); }
    else if (out_type == BW_BF16) { if (vec) BW_RS(bf16, 4); else BW_RS(bf16, 1); }
    else return BW_ERR_BAD_ARG;
#undef BW_RS
    BW_LAUNCH_CHECK();
    return 0;
}

// out [T, 2H] of out_type = (a | b), both float32 [T, H].
BW_EXPORT int bw_concat2_cast(const float* a, const float* b, void* out, int out_type, int T, int H, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out);
    const int threads = H >= 1024 ? 256 : 128;
#define BW_CC(OT, W) bw::launch((concat2_cast_kernel<OT, W>), dim3(T), dim3(threads), 0, s, a, b, (OT*)out, H)
    if (out_type == BW_F32) { if (vec) BW_CC(float, 4); else BW_CC(float, 1); }
    else if (out_type == BW_BF16) { if (vec) BW_CC(bf16, 4); else BW_CC(bf16, 1); }
    else return BW_ERR_BAD_ARG;
#undef BW_CC
    BW_LAUNCH_CHECK();
    return 0;
}
