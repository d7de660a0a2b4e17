// Query/key norm over the whole projection, rotary encoding and cache append in one kernel, for
// attention mixers whose q/k/v projection cannot carry the rotation in its own epilogue (the norm
// needs the whole row first) and whose heads may have a key size different from the value size.
//
// qkv: float32 [T, nh*dq + nkv*dq + nkv*dv] (queries, keys, values; biases already added).
//   * norm (optional, q_gain/k_gain non-null): all nh*dq query channels of a token are divided by their
//     common root mean square and multiplied by a gain per channel; the same for the nkv*dq key channels.
//   * rotation of the first rotary_dim channels of every q and k head with the step's cos/sin table
//     [T, rotary_dim] (cosines, then sines; any magnitude factor is already in the table).
//     interleaved != 0: channel 2i pairs with 2i + 1; else channel i pairs with i + rotary_dim / 2.
//   * q_out [T, nh, dpad], keys and values to the page of the token's position,
//     pages [num_pages, nkv, page_size, dpad]; channels from dq (dv) up to dpad are written as zeros, so
//     that an attention kernel built for one head size serves both.
// All arithmetic is float32; one block per token.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

template <typename OT>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                    const int* __restrict__ req_of_token, const int* __restrict__ block_table, int max_blocks,
                    const float* __restrict__ table, int rotary_dim, int interleaved,
                    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                    OT* __restrict__ q_out, OT* __restrict__ k_pages, OT* __restrict__ v_pages,
                    int nh, int nkv, int dq, int dv, int dpad, int page_size, int num_pages) {
    BW_PDL_TRIGGER();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int nq = nh * dq, nk = nkv * dq, nv = nkv * dv;
    const int pos = positions[t];
    int page = -1;
    const int slot = pos % page_size;
    if (num_pages > 0) {
        page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page >= num_pages) page = -1;
    }
    BW_PDL_WAIT();
    const float* row = qkv + (size_t)t * (nq + nk + nv);
    float rq = 1.f, rk = 1.f;
    if (q_gain) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = row[c]; ss = fmaf(v, v, ss); }
        rq = rsqrtf(bw::block_sum(ss, scratch) / (float)nq + eps);
    }
    if (k_gain) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = row[nq + c]; ss = fmaf(v, v, ss); }
        rk = rsqrtf(bw::block_sum(ss, scratch) / (float)nk + eps);
    }
    const int half = rotary_dim >> 1;
    const float* tab = table + (size_t)t * rotary_dim;
    // queries and keys: heads 0..nh-1 are queries, nh..nh+nkv-1 keys
    const int n_qk = (nh + nkv) * dpad;
    for (int idx = threadIdx.x; idx < n_qk; idx += blockDim.x) {
        const int h = idx / dpad, c = idx - h * dpad;
        const bool is_q = h < nh;
        float o = 0.f;
        if (c < dq) {
            const float* src = is_q ? row + (size_t)h * dq : row + nq + (size_t)(h - nh) * dq;
            const float* gain = is_q ? (q_gain ? q_gain + (size_t)h * dq : nullptr)
                                     : (k_gain ? k_gain + (size_t)(h - nh) * dq : nullptr);
            const float r = is_q ? rq : rk;
            float x = src[c] * r;
            if (gain) x *= gain[c];
            o = x;
            if (c < rotary_dim) {
                int j, pc; bool first;
                if (interleaved) { j = c >> 1; pc = c ^ 1; first = !(c & 1); }
                else { first = c < half; j = first ? c : c - half; pc = first ? c + half : c - half; }
                float y = src[pc] * r;
                if (gain) y *= gain[pc];
                const float cs = tab[j], sn = tab[half + j];
                o = first ? x * cs - y * sn : x * cs + y * sn;
            }
        }
        if (is_q) q_out[((size_t)t * nh + h) * dpad + c] = bw::from_f32<OT>(o);
        else if (page >= 0) k_pages[(((size_t)page * nkv + (h - nh)) * page_size + slot) * dpad + c] = bw::from_f32<OT>(o);
    }
    if (page >= 0) {
        const float* vsrc = row + nq + nk;
        for (int idx = threadIdx.x; idx < nkv * dpad; idx += blockDim.x) {
            const int h = idx / dpad, c = idx - h * dpad;
            const float o = c < dv ? vsrc[(size_t)h * dv + c] : 0.f;
            v_pages[(((size_t)page * nkv + h) * page_size + slot) * dpad + c] = bw::from_f32<OT>(o);
        }
    }
}

__device__ __forceinline__ void put4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void put4(bf16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(bw::pack_bf16x2(v.x, v.y), bw::pack_bf16x2(v.z, v.w));
}

// The same with the norm taken per HEAD: every query head of dq channels is divided by its own root mean
// square and multiplied by q_gain [dq], one gain vector shared by all heads (k_gain [dq] for the key heads);
// a null gain: no norm on that side.  After norm and rotation the queries of a token at position p are
// multiplied by  1 + q_coef * log(1 + n), n = whole periods of q_every positions in p + 1,   (q_coef == 0: by nothing), a temperature that
// grows with the logarithm of the position.  Rows of qkv are `ld` floats apart and hold the queries first,
// then (has_kv != 0) keys and values; whatever follows in the row (a gate's projection) is not touched.
// has_kv == 0: a run that reads another run's keys and values projects none.  One block per token, one warp
// per head at a time; all arithmetic float32.  v_first != null: the values become (1 - lam) v + lam v_first on their way
// into the cache, v_first being float32 rows `v_first_ld` apart with nkv * dv values of the same token (another layer's
// values of this step) and lam = *v_lam a number on the device.
template <typename OT>
__global__ void __launch_bounds__(256)
head_norm_rope_kernel(const float* __restrict__ qkv, long long ld, const int* __restrict__ positions,
                      const int* __restrict__ req_of_token, const int* __restrict__ block_table, int max_blocks,
                      const float* __restrict__ table, int rotary_dim, int interleaved,
                      const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                      float q_coef, float q_every,
                      OT* __restrict__ q_out, OT* __restrict__ k_pages, OT* __restrict__ v_pages,
                      int nh, int nkv, int dq, int dv, int dpad, int page_size, int num_pages, int has_kv, int vec,
                      float v_eps, const float* __restrict__ v_first, long long v_first_ld, const float* __restrict__ v_lam) {
    BW_PDL_TRIGGER();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int nq = nh * dq, nk = nkv * dq;
    const int pos = positions[t];
    int page = -1;
    const int slot = pos % page_size;
    if (has_kv && num_pages > 0) {
        page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page >= num_pages) page = -1;
    }
    float q_mult = 1.f;
    if (q_coef != 0.f) q_mult = 1.f + q_coef * logf((float)floor((double)(pos + 1) / (double)q_every) + 1.f);
    BW_PDL_WAIT();
    const float* row = qkv + (size_t)t * ld;
    const int half = rotary_dim >> 1;
    const float* tab = rotary_dim ? table + (size_t)t * rotary_dim : nullptr;
    const int n_heads = nh + (has_kv ? nkv : 0);
    for (int h = warp; h < n_heads; h += nwarps) {
        const bool is_q = h < nh;
        if (!is_q && page < 0) continue;
        const float* src = is_q ? row + (size_t)h * dq : row + nq + (size_t)(h - nh) * dq;
        const float* gain = is_q ? q_gain : k_gain;
        float r = 1.f;
        if (gain) {
            float ss = 0.f;
            for (int c = lane; c < dq; c += 32) { const float v = src[c]; ss = fmaf(v, v, ss); }
            r = rsqrtf(bw::warp_sum(ss) / (float)dq + eps);
        }
        const float mult = is_q ? q_mult : 1.f;
        OT* dst = is_q ? q_out + ((size_t)t * nh + h) * dpad
                       : k_pages + (((size_t)page * nkv + (h - nh)) * page_size + slot) * dpad;
        if (vec) {
            // no rotation, sizes that are multiples of 4, aligned rows: four channels a lane, 16-byte loads
            for (int c = lane * 4; c < dpad; c += 128) {
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < dq) {
                    o = *reinterpret_cast<const float4*>(src + c);
                    const float4 g = gain ? *reinterpret_cast<const float4*>(gain + c) : make_float4(1.f, 1.f, 1.f, 1.f);
                    o.x = o.x * r * g.x * mult; o.y = o.y * r * g.y * mult; o.z = o.z * r * g.z * mult; o.w = o.w * r * g.w * mult;
                }
                put4(dst + c, o);
            }
            continue;
        }
        for (int c = lane; c < dpad; c += 32) {
            float o = 0.f;
            if (c < dq) {
                float x = src[c] * r;
                if (gain) x *= gain[c];
                o = x;
                if (c < rotary_dim) {
                    int j, pc; bool first;
                    if (interleaved) { j = c >> 1; pc = c ^ 1; first = !(c & 1); }
                    else { first = c < half; j = first ? c : c - half; pc = first ? c + half : c - half; }
                    float y = src[pc] * r;
                    if (gain) y *= gain[pc];
                    const float cs = tab[j], sn = tab[half + j];
                    o = first ? x * cs - y * sn : x * cs + y * sn;
                }
                o *= mult;
            }
            dst[c] = bw::from_f32<OT>(o);
        }
    }
    // a value as it is cached: mixed with the same token's value of another layer where the launch says so
    const float* vsrc = row + nq + nk;
    const float* vf = v_first ? v_first + (size_t)t * v_first_ld : nullptr;
    const float lam = v_first ? *v_lam : 0.f;
    auto value = [&](size_t i) { const float v = vsrc[i]; return vf ? (1.f - lam) * v + lam * vf[i] : v; };
    if (page >= 0 && v_eps > 0.f) {
        // every value head divided by its own root mean square (no gain): a warp per head
        for (int h = warp; h < nkv; h += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < dv; c += 32) { const float v = value((size_t)h * dv + c); ss = fmaf(v, v, ss); }
            const float r = rsqrtf(bw::warp_sum(ss) / (float)dv + v_eps);
            OT* dst = v_pages + (((size_t)page * nkv + h) * page_size + slot) * dpad;
            for (int c = lane; c < dpad; c += 32) dst[c] = bw::from_f32<OT>(c < dv ? value((size_t)h * dv + c) * r : 0.f);
        }
        return;
    }
    if (page >= 0) {
        if (vec && !vf) {
            for (int idx = threadIdx.x * 4; idx < nkv * dpad; idx += blockDim.x * 4) {
                const int h = idx / dpad, c = idx - h * dpad;
                const float4 o = c < dv ? *reinterpret_cast<const float4*>(vsrc + (size_t)h * dv + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                put4(v_pages + (((size_t)page * nkv + h) * page_size + slot) * dpad + c, o);
            }
            return;
        }
        for (int idx = threadIdx.x; idx < nkv * dpad; idx += blockDim.x) {
            const int h = idx / dpad, c = idx - h * dpad;
            const float o = c < dv ? value((size_t)h * dv + c) : 0.f;
            v_pages[(((size_t)page * nkv + h) * page_size + slot) * dpad + c] = bw::from_f32<OT>(o);
        }
    }
}

}  // namespace

// The per-head form (head_norm_rope_kernel).  ld: floats between rows of qkv; q_gain / k_gain: float32 [dq] or
// null; q_coef, q_every: the queries' temperature (q_coef == 0: none; q_every > 0); has_kv == 0: the rows hold
// no keys and values and nothing is appended.  v_eps > 0: every value head is divided by sqrt(mean(v^2) + v_eps) on its way
// into the cache.  v_first, v_first_ld, v_lam: the value mixing (see the kernel), or nulls.
BW_EXPORT int bw_head_norm_rope_append(const float* qkv, long long ld, const int* positions, const int* req_of_token,
                                       const int* block_table, int max_blocks, const float* table, int rotary_dim,
                                       int interleaved, const float* q_gain, const float* k_gain, float eps,
                                       float q_coef, float q_every, void* q_out, void* k_pages, void* v_pages,
                                       int out_type, int T, int nh, int nkv, int dq, int dv, int dpad, int page_size,
                                       int num_pages, int has_kv, float v_eps, const float* v_first, long long v_first_ld,
                                       const float* v_lam, void* stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dq || (rotary_dim & 1) || dq <= 0 || dv <= 0 || dpad < dq || dpad < dv ||
        nh <= 0 || nkv <= 0 || page_size <= 0 || (rotary_dim > 0 && !table) || (q_coef != 0.f && !(q_every > 0.f)) ||
        ld < (long long)nh * dq + (has_kv ? (long long)nkv * (dq + dv) : 0) ||
        (v_first && (!v_lam || !has_kv || v_first_ld < (long long)nkv * dv)))
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = rotary_dim == 0 && (dq & 3) == 0 && (dv & 3) == 0 && (dpad & 3) == 0 && (ld & 3) == 0 &&
                    (((uintptr_t)qkv | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
#define BW_HN(OT) bw::launch((head_norm_rope_kernel<OT>), dim3(T), dim3(256), 0, s, qkv, ld, positions, req_of_token, block_table, \
        max_blocks, table, rotary_dim, interleaved, q_gain, k_gain, eps, q_coef, q_every, (OT*)q_out, (OT*)k_pages, (OT*)v_pages, \
        nh, nkv, dq, dv, dpad, page_size, num_pages, has_kv, vec, v_eps, v_first, v_first_ld, v_lam)
    if (out_type == BW_F32) BW_HN(float);
    else if (out_type == BW_BF16) BW_HN(bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_HN
    BW_LAUNCH_CHECK();
    return 0;
}

// out_type: element type of q_out and the pages.  num_pages <= 0: nothing is appended (a run that reads
// another run's cache).  q_gain / k_gain: float32 gains of the norm, or null for no norm.
BW_EXPORT int bw_qk_norm_rope_append(const float* qkv, const int* positions, const int* req_of_token,
                                     const int* block_table, int max_blocks, const float* table, int rotary_dim,
                                     int interleaved, const float* q_gain, const float* k_gain, float eps,
                                     void* q_out, void* k_pages, void* v_pages, int out_type, int T, int nh, int nkv,
                                     int dq, int dv, int dpad, int page_size, int num_pages, void* stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dq || (rotary_dim & 1) || dq <= 0 || dv <= 0 || dpad < dq || dpad < dv ||
        nh <= 0 || nkv <= 0 || page_size <= 0 || (rotary_dim > 0 && !table))
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
#define BW_QK(OT) bw::launch((qk_norm_rope_kernel<OT>), dim3(T), dim3(256), 0, s, qkv, positions, req_of_token, block_table, \
        max_blocks, table, rotary_dim, interleaved, q_gain, k_gain, eps, (OT*)q_out, (OT*)k_pages, (OT*)v_pages, nh, nkv, dq, dv, \
        dpad, page_size, num_pages)
    if (out_type == BW_F32) BW_QK(float);
    else if (out_type == BW_BF16) BW_QK(bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_QK
    BW_LAUNCH_CHECK();
    return 0;
}
