// Memory-bound row kernels: embedding gather, RMSNorm (optionally on gathered rows),
// SwiGLU, and rotary position encoding fused with the append of keys and values
// into cache pages.  All arithmetic is 32-bit; inputs and outputs are float32 or
// bfloat16 as the type codes say.  Any width is accepted (no power-of-two rule).
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

// ---------------------------------------------------------------- embedding
template <typename WT>
__global__ void embed_gather_kernel(const WT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, float scale) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) id = 0;  // the host rejects such ids before the launch
    const WT* row = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    const int c0 = blockIdx.y * blockDim.x * 4;   // each block copies 4 * blockDim elements of the row
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * blockDim.x + threadIdx.x;
        if (c < H) o[c] = bw::to_f32(row[c]) * scale;   // scale 1: the stored value
    }
}

// The same with a sine/cosine vector of the token's position added, written `copies` times side by side
// (out [T, copies, H]): entry 2i is sin(pos * inv_freq[i]), entry 2i + 1 the cosine of the same angle.  The
// angle is the float32 product of the position and the frequency; sine and cosine are the precise ones.
// inv_freq == null: no position vector.
template <typename WT>
__global__ void embed_positions_kernel(const WT* __restrict__ table, const int* __restrict__ ids,
                                       const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                       float* __restrict__ out, int H, int V, float scale, int copies) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) id = 0;  // the host rejects such ids before the launch
    const WT* row = table + (size_t)id * H;
    float* o = out + (size_t)t * copies * H;
    const float pos = (float)positions[t];
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = bw::to_f32(row[c]) * scale;
        if (inv_freq) {
            const float ang = pos * inv_freq[c >> 1];
            v += (c & 1) ? cosf(ang) : sinf(ang);
        }
        for (int k = 0; k < copies; ++k) o[(size_t)k * H + c] = v;
    }
}

// ---------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w.  One block per output row; input row is
// rows[i] when `rows` is given (final norm on the rows whose logits are wanted).
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const WT* __restrict__ w,
                               const int* __restrict__ rows, OT* __restrict__ out,
                               int H, float eps, long long ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    const float* xr = x + (size_t)src * (size_t)ld;
    OT* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) { float v = xr[c]; ss = fmaf(v, v, ss); }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        o[c] = bw::from_f32<OT>(xr[c] * r * bw::to_f32(w[c]));
}

// The same with 4 elements per access, for widths that are multiples of 4 (the sum runs over
// the same per-thread strided order scaled by 4; rows stay independent of one another).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a); r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename WT, typename OT>
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, const WT* __restrict__ w,
                                    const int* __restrict__ rows, OT* __restrict__ out, int H, float eps, long long ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    const float* xr = x + (size_t)src * (size_t)ld;
    OT* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        const float4 v = load4(xr + c);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
        const float4 v = load4(xr + c), g = load4(w + c);
        store4(o + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
    }
}

// v += p[0] + p[stride] + ... (n values, added in that order; four loads in flight at a time)
__device__ __forceinline__ void add_planes4(float4& v, const float* p, int n, size_t stride) {
    for (int p0 = 0; p0 < n; p0 += 4) {
        float4 t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = p0 + j < n ? load4(p + (size_t)(p0 + j) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) { v.x += t[j].x; v.y += t[j].y; v.z += t[j].z; v.w += t[j].w; }
    }
}
__device__ __forceinline__ void add_planes1(float& v, const float* p, int n, size_t stride) {
    for (int p0 = 0; p0 < n; p0 += 4) {
        float t[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = p0 + j < n ? p[(size_t)(p0 + j) * stride] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) v += t[j];
    }
}

// x += planes[0] + planes[1] + ... (in that order), then the norm of the new x: the planes are a matrix
// product that its kernel left unsummed (bw_gemm_tc_planes).  One block per output row.  With
// `rows` (the final norm on chosen rows, which may repeat) x is left as it is and only the norm's
// input is the sum.  Every thread re-reads only what it wrote itself.
template <typename WT, typename OT, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes,
                                   size_t plane_stride, const WT* __restrict__ w, const int* __restrict__ rows,
                                   OT* __restrict__ out, int H, float eps) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    float* xr = x + (size_t)src * H;
    const float* pr = planes + (size_t)src * H;
    OT* o = out + (size_t)i * H;
    constexpr int W = VEC ? 4 : 1;
    float ss = 0.f;
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            float4 v = load4(xr + c);
            add_planes4(v, pr + c, n_planes, plane_stride);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            if (!rows) store4(xr + c, v);
        } else {
            float v = xr[c];
            add_planes1(v, pr + c, n_planes, plane_stride);
            ss = fmaf(v, v, ss);
            if (!rows) xr[c] = v;
        }
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            float4 v = load4(xr + c);
            if (rows) add_planes4(v, pr + c, n_planes, plane_stride);
            const float4 g = load4(w + c);
            store4(o + c, make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w));
        } else {
            float v = xr[c];
            if (rows) add_planes1(v, pr + c, n_planes, plane_stride);
            o[c] = bw::from_f32<OT>(v * r * bw::to_f32(w[c]));
        }
    }
}

// x += planes[0] + planes[1] + ... (in that order)
__global__ void add_planes_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes,
                                  size_t plane_stride, size_t total) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        add_planes1(v, planes + i, n_planes, plane_stride);
        x[i] = v;
    }
}

// x = planes[0] + planes[1] + ... (in that order): a product that was WRITTEN as planes, not added
__global__ void sum_planes_kernel(float* __restrict__ x, const float* __restrict__ planes, int n_planes,
                                  size_t plane_stride, size_t total) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        add_planes1(v, planes + i, n_planes, plane_stride);
        x[i] = v;
    }
}

// x[t, c] += a[t, c] * ga[c] (+ b[t, c] * gb[c]): sublayers' outputs, each times a gain per channel ("layer scale"),
// summed and added to the stream.  The two products are added to each other first, then to x.
__global__ void scale_add_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ ga,
                                 const float* __restrict__ b, const float* __restrict__ gb, size_t total, int H) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % (size_t)H);
        float y = a[i] * ga[c];
        if (b) y += b[i] * gb[c];
        x[i] += y;
    }
}

// The same sum and, in the same pass over the row, two RMS norms of the new row with a gain each (a block whose two
// sublayers read two norms of the same stream): x[t] += a[t] * ga + b[t] * gb (a == null: x stays as it is), then
// o1[t] = x[t] / rms(x[t]) * w1 and (o2 != null) o2[t] = x[t] / rms(x[t]) * w2.  One block per row; every thread re-reads
// only what it wrote itself; the order of the sum of squares depends on H and the block size alone.
template <typename WT, typename OT, bool VEC>
__global__ void scale_add_norm2_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ ga,
                                       const float* __restrict__ b, const float* __restrict__ gb,
                                       const WT* __restrict__ w1, const WT* __restrict__ w2, OT* __restrict__ o1,
                                       OT* __restrict__ o2, const int* __restrict__ rows, int H, float eps1, float eps2) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    // rows != null: only these rows are read (x stays as it is: the stream ends here), the results are dense
    const size_t row = (size_t)(rows ? rows[blockIdx.x] : (int)blockIdx.x) * H, orow = (size_t)blockIdx.x * H;
    float* xr = x + row;
    constexpr int W = VEC ? 4 : 1;     // VEC: four channels a thread and access (H a multiple of 4, 16-byte aligned rows)
    auto sum4 = [&](int c) {           // the new row's four channels from c on
        float4 v = load4(xr + c);
        if (a) {
            const float4 av = load4(a + row + c), g1 = load4(ga + c);
            float4 y = make_float4(av.x * g1.x, av.y * g1.y, av.z * g1.z, av.w * g1.w);
            if (b) {
                const float4 bv = load4(b + row + c), g2 = load4(gb + c);
                y.x += bv.x * g2.x; y.y += bv.y * g2.y; y.z += bv.z * g2.z; y.w += bv.w * g2.w;
            }
            v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
        }
        return v;
    };
    auto sum1 = [&](int c) {
        float v = xr[c];
        if (a) {
            float y = a[row + c] * ga[c];
            if (b) y += b[row + c] * gb[c];
            v += y;
        }
        return v;
    };
    float ss = 0.f;
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            const float4 v = sum4(c);
            if (a && !rows) store4(xr + c, v);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        } else {
            const float v = sum1(c);
            if (a && !rows) xr[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = bw::block_sum(ss, scratch) / (float)H;
    const float r1 = rsqrtf(ss + eps1), r2 = rsqrtf(ss + eps2);
    for (int c = threadIdx.x * W; c < H; c += blockDim.x * W) {
        if constexpr (VEC) {
            const float4 v = rows ? sum4(c) : load4(xr + c), g1 = load4(w1 + c);
            store4(o1 + orow + c, make_float4(v.x * r1 * g1.x, v.y * r1 * g1.y, v.z * r1 * g1.z, v.w * r1 * g1.w));
            if (o2) {
                const float4 g2 = load4(w2 + c);
                store4(o2 + orow + c, make_float4(v.x * r2 * g2.x, v.y * r2 * g2.y, v.z * r2 * g2.z, v.w * r2 * g2.w));
            }
        } else {
            const float v = rows ? sum1(c) : xr[c];
            o1[orow + c] = bw::from_f32<OT>(v * r1 * bw::to_f32(w1[c]));
            if (o2) o2[orow + c] = bw::from_f32<OT>(v * r2 * bw::to_f32(w2[c]));
        }
    }
}

// ---------------------------------------------------------------- SwiGLU and other activations
// in: [T, 2I] with gate in columns [0, I) and up in [I, 2I); out: [T, I] = bw::glu(act, gate, up, limit, alpha)
// (BW_ACT_SILU: silu(gate) * up).
template <typename IT, typename OT>
__global__ void swiglu_kernel(const IT* __restrict__ gu, OT* __restrict__ out, int I, size_t total, int act, float limit,
                              float alpha) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I; const int c = (int)(idx - t * I);
        const float g = bw::to_f32(gu[t * 2 * (size_t)I + c]);
        const float u = bw::to_f32(gu[t * 2 * (size_t)I + I + c]);
        out[idx] = bw::from_f32<OT>(bw::glu(act, g, u, limit, alpha));
    }
}

// An activation without a gate, element by element: BW_ACT_RELU2: max(x, 0)^2.
template <typename IT, typename OT>
__global__ void unary_act_kernel(const IT* __restrict__ x, OT* __restrict__ out, size_t total, int act) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = bw::from_f32<OT>(bw::unary_act(act, bw::to_f32(x[idx])));
}

// o[t, h, c] *= sigmoid(g[t, h * dv + c]) for c < dv (o has dpad >= dv channels a head; those beyond dv become 0):
// the output gate of a mixer.  g: float32 rows `ld` apart.  One block per token.
template <typename OT>
__global__ void sigmoid_gate_kernel(OT* __restrict__ o, const float* __restrict__ g, long long ld, int nh, int dv, int dpad) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    OT* orow = o + (size_t)blockIdx.x * nh * dpad;
    const float* grow = g + (size_t)blockIdx.x * ld;
    for (int idx = threadIdx.x; idx < nh * dpad; idx += blockDim.x) {
        const int h = idx / dpad, c = idx - h * dpad;
        float v = 0.f;
        if (c < dv) v = bw::to_f32(orow[idx]) / (1.f + expf(-grow[(size_t)h * dv + c]));
        orow[idx] = bw::from_f32<OT>(v);
    }
}

// ---------------------------------------------------------------- RoPE + append
// qkv: [T, (nh + 2 nkv) * hd] (q heads, then k heads, then v heads).
// q_out: [T, nh * hd] rotated queries.  Rotated keys and raw values go to the
// page of the token's position: pages are [num_pages, nkv, page_size, hd].
// rotary_dim = 0 rotates nothing (a mixer without rotary encoding).
// cos and sin of pos * inv_freq[j] for every token of the step: [T, rotary_dim] (cos, then sin).
// All layers with the same rotary parameters share one table per step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ table, int rotary_dim, int T, float magnitude) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int half = rotary_dim >> 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, j = idx - t * half;
    float s, c;
    sincosf((float)positions[t] * inv_freq[j], &s, &c);
    table[(size_t)t * rotary_dim + j] = c * magnitude;
    table[(size_t)t * rotary_dim + half + j] = s * magnitude;
}

// Where each token of the step keeps its keys and values: page * page_size + slot of its position,
// or -1 when the block table names no page there.  The same for all layers of a cache group.
__global__ void kv_slots_kernel(const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages,
                                int* __restrict__ kv_slot, int T) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
    kv_slot[t] = (page >= 0 && page < num_pages) ? page * page_size + pos % page_size : -1;
}

constexpr int ROPE_HPB = 8;   // heads per block of rope_append_kernel

template <typename IT, typename OT>
__global__ void rope_append_kernel(const IT* __restrict__ qkv, const int* __restrict__ positions,
                                   const int* __restrict__ req_of_token,
                                   const int* __restrict__ block_table, int max_blocks,
                                   const float* __restrict__ inv_freq, const float* __restrict__ table,
                                   int rotary_dim, OT* __restrict__ q_out, OT* __restrict__ k_pages,
                                   OT* __restrict__ v_pages, int nh, int nkv, int hd,
                                   int page_size, int num_pages, int paired, int n_planes, size_t plane_stride) {
    BW_PDL_TRIGGER();
    // A block takes ROPE_HPB heads of one token; a thread takes one channel of each of them: the
    // loads of the heads are independent and in flight together, the angle is looked up once.
    // Positions and block tables were on the device before the step's first kernel ran, so the page
    // is looked up before the wait for the kernels that make qkv and the table.
    const int t = blockIdx.x, h0 = blockIdx.y * ROPE_HPB;
    const int n_heads = nh + 2 * nkv;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    const IT* row = qkv + (size_t)t * n_heads * hd;
    int page = -1, slot = 0;
    if (h0 + ROPE_HPB > nh) {   // this block holds key or value heads
        const int r = req_of_token[t];
        page = block_table[(size_t)r * max_blocks + pos / page_size];
        slot = pos % page_size;
        if (page >= num_pages) page = -1;
    }
    BW_PDL_WAIT();
    for (int c = threadIdx.x; c < hd; c += blockDim.x) {
        float sn = 0.f, cs = 1.f;
        const bool rot_c = c < rotary_dim;
        if (rot_c) {
            const int j = c < half ? c : c - half;
            if (table) { cs = table[(size_t)t * rotary_dim + j]; sn = table[(size_t)t * rotary_dim + half + j]; }
            else sincosf((float)pos * inv_freq[j], &sn, &cs);
            if (c < half) sn = -sn;   // first half: x cos - partner sin; second half: partner sin + x cos
        }
        // paired: in the q and k heads the input holds channel j and its partner j + half side by side
        // (at 2j and 2j + 1), the order the fused projection's weight rows have
        const int sc = (paired && rot_c) ? (c < half ? 2 * c : 2 * (c - half) + 1) : c;
        const int pc = rot_c ? (paired ? (sc ^ 1) : (c < half ? c + half : c - half)) : c;
        float v[ROPE_HPB], w[ROPE_HPB];
#pragma unroll
        for (int k = 0; k < ROPE_HPB; ++k) {
            const int h = h0 + k;
            v[k] = h < n_heads ? bw::to_f32(row[(size_t)h * hd + (h < nh + nkv ? sc : c)]) : 0.f;
            w[k] = (h < nh + nkv && rot_c) ? bw::to_f32(row[(size_t)h * hd + pc]) : 0.f;
        }
        // qkv left as planes by its matrix product: the further planes are added in order
        for (int p0 = 1; p0 < n_planes; p0 += 2) {   // two planes' loads in flight together
            float tv[2][ROPE_HPB], tw[2][ROPE_HPB];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const IT* prow = row + (size_t)(p0 + j) * plane_stride;
                const bool there = p0 + j < n_planes;
#pragma unroll
                for (int k = 0; k < ROPE_HPB; ++k) {
                    const int h = h0 + k;
                    tv[j][k] = (there && h < n_heads) ? bw::to_f32(prow[(size_t)h * hd + (h < nh + nkv ? sc : c)]) : 0.f;
                    tw[j][k] = (there && h < nh + nkv && rot_c) ? bw::to_f32(prow[(size_t)h * hd + pc]) : 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int k = 0; k < ROPE_HPB; ++k) { v[k] += tv[j][k]; w[k] += tw[j][k]; }
            }
        }
#pragma unroll
        for (int k = 0; k < ROPE_HPB; ++k) {
            const int h = h0 + k;
            if (h >= n_heads) break;
            const float o = (h < nh + nkv && rot_c) ? v[k] * cs + w[k] * sn : v[k];
            if (h < nh) {
                q_out[((size_t)t * nh + h) * hd + c] = bw::from_f32<OT>(o);
            } else if (page >= 0) {
                const bool is_k = h < nh + nkv;
                const int kvh = is_k ? h - nh : h - nh - nkv;
                (is_k ? k_pages : v_pages)[(((size_t)page * nkv + kvh) * page_size + slot) * hd + c] = bw::from_f32<OT>(o);
            }
        }
    }
}

// ---------------------------------------------------------------- norm of a branch, added to the stream
// stream[i] += x[i] * rsqrt(mean(x[i]^2) + eps) * w  (the norm that FOLLOWS a sublayer); with w2 also
// out[i] = stream[i] * rsqrt(mean(stream[i]^2) + eps2) * w2, the norm BEFORE the next sublayer, in the same pass.
// One block per row; the row is read once (16-byte loads when the width allows) and kept in shared memory.
template <typename WT, typename OT, bool NEXT>
__global__ void rmsnorm_add_kernel(const float* __restrict__ x, const WT* __restrict__ w, float* __restrict__ stream,
                                   const WT* __restrict__ w2, OT* __restrict__ out, int H, float eps, float eps2) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    extern __shared__ __align__(16) float row[];   // [H]: x, then the new stream values
    __shared__ float scratch[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float* sr = stream + (size_t)blockIdx.x * H;
    const bool vec = (H & 3) == 0;
    float ss = 0.f;
    if (vec) {
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
            const float4 v = load4(xr + c);
            store4(row + c, v);
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = xr[c]; row[c] = v; ss = fmaf(v, v, ss); }
    }
    ss = bw::block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    float ss2 = 0.f;
    if (vec) {
        for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {   // each thread reads back what it wrote
            const float4 v = load4(row + c), g = load4(w + c);
            float4 o = load4(sr + c);
            o.x += v.x * r * g.x; o.y += v.y * r * g.y; o.z += v.z * r * g.z; o.w += v.w * r * g.w;
            store4(sr + c, o);
            if (NEXT) { store4(row + c, o); ss2 = fmaf(o.x, o.x, ss2); ss2 = fmaf(o.y, o.y, ss2); ss2 = fmaf(o.z, o.z, ss2); ss2 = fmaf(o.w, o.w, ss2); }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float o = sr[c] + row[c] * r * bw::to_f32(w[c]);
            sr[c] = o;
            if (NEXT) { row[c] = o; ss2 = fmaf(o, o, ss2); }
        }
    }
    if (NEXT) {
        ss2 = bw::block_sum(ss2, scratch);
        const float r2 = rsqrtf(ss2 / (float)H + eps2);
        OT* o = out + (size_t)blockIdx.x * H;
        if (vec) {
            for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
                const float4 v = load4(row + c), g = load4(w2 + c);
                store4(o + c, make_float4(v.x * r2 * g.x, v.y * r2 * g.y, v.z * r2 * g.z, v.w * r2 * g.w));
            }
        } else {
            for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = bw::from_f32<OT>(row[c] * r2 * bw::to_f32(w2[c]));
        }
    }
}

// ---------------------------------------------------------------- logits
// In place: x * scale, then cap * tanh(x / cap) when cap > 0 (a model's logit multiplier and soft cap).
__global__ void logit_transform_kernel(float* __restrict__ x, long long n, float scale, float cap) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v * inv_cap);
        x[i] = v;
    }
}

template <typename T> const T* cp(const void* p) { return reinterpret_cast<const T*>(p); }
template <typename T> T* mp(void* p) { return reinterpret_cast<T*>(p); }

}  // namespace

BW_EXPORT int bw_logit_transform(float* logits, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    bw::launch(logit_transform_kernel, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(threads), 0,
               (cudaStream_t)stream, logits, n, scale, cap);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_embed_gather(const void* table, int table_type, const int* ids, float* out,
                              int T, int H, int V, float scale, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    const dim3 grid(T, (H + threads * 4 - 1) / (threads * 4));
    if (table_type == BW_F32) bw::launch((embed_gather_kernel<float>), dim3(grid), dim3(threads), 0, s, cp<float>(table), ids, out, H, V, scale);
    else if (table_type == BW_BF16) bw::launch((embed_gather_kernel<bf16>), dim3(grid), dim3(threads), 0, s, cp<bf16>(table), ids, out, H, V, scale);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// out float32 [T, copies, H]; inv_freq float32 [ceil(H / 2)] or null (no position vector)
BW_EXPORT int bw_embed_positions(const void* table, int table_type, const int* ids, const int* positions,
                                 const float* inv_freq, float* out, int T, int H, int V, float scale, int copies, void* stream) {
    if (T <= 0) return 0;
    if (copies <= 0 || H <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_type == BW_F32) bw::launch((embed_positions_kernel<float>), dim3(T), dim3(threads), 0, s, cp<float>(table), ids, positions, inv_freq, out, H, V, scale, copies);
    else if (table_type == BW_BF16) bw::launch((embed_positions_kernel<bf16>), dim3(T), dim3(threads), 0, s, cp<bf16>(table), ids, positions, inv_freq, out, H, V, scale, copies);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// the rows of x lie `ld` floats apart (ld >= H: x may be a range of columns of a wider tensor); out is dense
BW_EXPORT int bw_rmsnorm_ld(const float* x, long long ld, const void* w, int w_type, const int* rows, void* out,
                            int out_type, int n_rows, int H, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    if (ld < H) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && ld % 4 == 0 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define BW_RMS(WT, OT) do { if (vec) bw::launch((rmsnorm_vec4_kernel<WT, OT>), dim3(n_rows), dim3(threads), 0, s, x, cp<WT>(w), rows, mp<OT>(out), H, eps, ld); \
        else bw::launch((rmsnorm_kernel<WT, OT>), dim3(n_rows), dim3(threads), 0, s, x, cp<WT>(w), rows, mp<OT>(out), H, eps, ld); } while (0)
    if (w_type == BW_F32 && out_type == BW_F32) BW_RMS(float, float);
    else if (w_type == BW_F32 && out_type == BW_BF16) BW_RMS(float, bf16);
    else if (w_type == BW_BF16 && out_type == BW_F32) BW_RMS(bf16, float);
    else if (w_type == BW_BF16 && out_type == BW_BF16) BW_RMS(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_RMS
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_rmsnorm(const float* x, const void* w, int w_type, const int* rows, void* out,
                         int out_type, int n_rows, int H, float eps, void* stream) {
    return bw_rmsnorm_ld(x, H, w, w_type, rows, out, out_type, n_rows, H, eps, stream);
}

// x[n_rows or more, H] += the planes (float32, plane_stride floats apart), out = rmsnorm of the new x.
// rows != null: out row i is the norm of x[rows[i]] + planes[.][rows[i]], and x is NOT changed.
BW_EXPORT int bw_add_rmsnorm(float* x, const float* planes, int n_planes, long long plane_stride, const void* w,
                             int w_type, const int* rows, void* out, int out_type, int n_rows, int H, float eps,
                             void* stream) {
    if (n_rows <= 0) return 0;
    if (!planes || n_planes < 1 || plane_stride < 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && plane_stride % 4 == 0 &&
                     (((uintptr_t)x | (uintptr_t)planes | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    // one pass over the row: a thread per four elements (up to 1,024 threads), so that the loads of
    // the stream and of all planes are in flight at once
    const int quads = (H / 4 + 31) / 32 * 32;
    const int threads = vec ? (quads > 1024 ? 1024 : (quads < 128 ? 128 : quads)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define BW_ARMS(WT, OT) do { if (vec) bw::launch((add_rmsnorm_kernel<WT, OT, true>), dim3(n_rows), dim3(threads), 0, s, x, planes, n_planes, (size_t)plane_stride, cp<WT>(w), rows, mp<OT>(out), H, eps); \
        else bw::launch((add_rmsnorm_kernel<WT, OT, false>), dim3(n_rows), dim3(threads), 0, s, x, planes, n_planes, (size_t)plane_stride, cp<WT>(w), rows, mp<OT>(out), H, eps); } while (0)
    if (w_type == BW_F32 && out_type == BW_F32) BW_ARMS(float, float);
    else if (w_type == BW_F32 && out_type == BW_BF16) BW_ARMS(float, bf16);
    else if (w_type == BW_BF16 && out_type == BW_F32) BW_ARMS(bf16, float);
    else if (w_type == BW_BF16 && out_type == BW_BF16) BW_ARMS(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_ARMS
    BW_LAUNCH_CHECK();
    return 0;
}

// x[total] += the planes, added in plane order
namespace {
template <typename WT, typename OT, bool NEXT>
int launch_rmsnorm_add(const float* x, const void* w, float* stream_rows, const void* w2, void* out, int n, int H, float eps,
                       float eps2, cudaStream_t s) {
    static bool raised[bw::MAX_DEVICES] = {};
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 48 * 1024 && bw::allow_dynamic_smem(rmsnorm_add_kernel<WT, OT, NEXT>, 200 * 1024, raised) != cudaSuccess) return BW_ERR_DRIVER;
    const int threads = H >= 2048 ? 256 : 128;
    bw::launch((rmsnorm_add_kernel<WT, OT, NEXT>), dim3(n), dim3(threads), smem, s, x, (const WT*)w, stream_rows, (const WT*)w2, (OT*)out, H, eps, eps2);
    BW_LAUNCH_CHECK();
    return 0;
}
}  // namespace

BW_EXPORT int bw_rmsnorm_add(const float* x, const void* w, int w_type, float* stream_rows, int n, int H, float eps,
                             void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (w_type == BW_F32) return launch_rmsnorm_add<float, float, false>(x, w, stream_rows, nullptr, nullptr, n, H, eps, 0.f, s);
    if (w_type == BW_BF16) return launch_rmsnorm_add<bf16, bf16, false>(x, w, stream_rows, nullptr, nullptr, n, H, eps, 0.f, s);
    return BW_ERR_BAD_ARG;
}

// both gains of w_type; out of out_type
BW_EXPORT int bw_rmsnorm_add_norm(const float* x, const void* w, float* stream_rows, const void* w2, int w_type, void* out,
                                  int out_type, int n, int H, float eps, float eps2, void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 200 * 1024) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (w_type == BW_F32 && out_type == BW_F32) return launch_rmsnorm_add<float, float, true>(x, w, stream_rows, w2, out, n, H, eps, eps2, s);
    if (w_type == BW_F32 && out_type == BW_BF16) return launch_rmsnorm_add<float, bf16, true>(x, w, stream_rows, w2, out, n, H, eps, eps2, s);
    if (w_type == BW_BF16 && out_type == BW_BF16) return launch_rmsnorm_add<bf16, bf16, true>(x, w, stream_rows, w2, out, n, H, eps, eps2, s);
    return BW_ERR_BAD_ARG;
}

BW_EXPORT int bw_add_planes(float* x, const float* planes, int n_planes, long long plane_stride, long long total,
                            void* stream) {
    if (total <= 0 || n_planes <= 0) return 0;
    if (!x || !planes || plane_stride < 0) return BW_ERR_BAD_ARG;
    const long long want = (total + 255) / 256;
    bw::launch(add_planes_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
               x, planes, n_planes, (size_t)plane_stride, (size_t)total);
    BW_LAUNCH_CHECK();
    return 0;
}

// x, a (and b, or null): float32 [T, H]; ga (gb): float32 [H]
BW_EXPORT int bw_scale_add(float* x, const float* a, const float* ga, const float* b, const float* gb, int T, int H,
                           void* stream) {
    if (T <= 0) return 0;
    if (!x || !a || !ga || H <= 0 || (b != nullptr) != (gb != nullptr)) return BW_ERR_BAD_ARG;
    const long long total = (long long)T * H, want = (total + 255) / 256;
    bw::launch(scale_add_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
               x, a, ga, b, gb, (size_t)total, H);
    BW_LAUNCH_CHECK();
    return 0;
}

// x, a, b: float32 [T, H] (a, or b alone, may be null); ga, gb: float32 [H]; w1, w2: gains of w_type; o1, o2 (o2 may be
// null): [n, H] of out_type.  rows: null (n = all T rows, x is updated) or n row numbers (x is left as it is).
BW_EXPORT int bw_scale_add_norm2(float* x, const float* a, const float* ga, const float* b, const float* gb, const void* w1,
                                 const void* w2, int w_type, void* o1, void* o2, int out_type, const int* rows, int T, int H,
                                 float eps1, float eps2, void* stream) {
    if (T <= 0) return 0;
    if (!x || !w1 || !o1 || H <= 0 || (a != nullptr) != (ga != nullptr) || (b != nullptr) != (gb != nullptr) || (b && !a) ||
        (o2 != nullptr) != (w2 != nullptr))
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)a | (uintptr_t)ga | (uintptr_t)b | (uintptr_t)gb | (uintptr_t)w1 |
                                     (uintptr_t)w2 | (uintptr_t)o1 | (uintptr_t)o2) & 15) == 0;
    const int threads = vec ? (H >= 4096 ? 512 : (H >= 1024 ? 256 : 128)) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define BW_SAN(WT, OT) do { if (vec) bw::launch((scale_add_norm2_kernel<WT, OT, true>), dim3(T), dim3(threads), 0, s, x, a, ga, b, gb, \
        (const WT*)w1, (const WT*)w2, (OT*)o1, (OT*)o2, rows, H, eps1, eps2); \
        else bw::launch((scale_add_norm2_kernel<WT, OT, false>), dim3(T), dim3(threads), 0, s, x, a, ga, b, gb, \
        (const WT*)w1, (const WT*)w2, (OT*)o1, (OT*)o2, rows, H, eps1, eps2); } while (0)
    if (w_type == BW_F32 && out_type == BW_F32) BW_SAN(float, float);
    else if (w_type == BW_F32 && out_type == BW_BF16) BW_SAN(float, bf16);
    else if (w_type == BW_BF16 && out_type == BW_F32) BW_SAN(bf16, float);
    else if (w_type == BW_BF16 && out_type == BW_BF16) BW_SAN(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_SAN
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_sum_planes(float* x, const float* planes, int n_planes, long long plane_stride, long long total,
                            void* stream) {
    if (total <= 0) return 0;
    if (!x || !planes || plane_stride < 0 || n_planes <= 0) return BW_ERR_BAD_ARG;
    const long long want = (total + 255) / 256;
    bw::launch(sum_planes_kernel, dim3((unsigned)(want < 148 * 8 ? want : 148 * 8)), dim3(256), 0, (cudaStream_t)stream,
               x, planes, n_planes, (size_t)plane_stride, (size_t)total);
    BW_LAUNCH_CHECK();
    return 0;
}

static int launch_glu(const void* gu, int in_type, void* out, int out_type, int T, int I, int act, float limit, float alpha, void* stream);

BW_EXPORT int bw_swiglu(const void* gu, int in_type, void* out, int out_type, int T, int I, void* stream) {
    return launch_glu(gu, in_type, out, out_type, T, I, BW_ACT_SILU, 0.f, 1.f, stream);
}

// act: a gated activation of common.cuh (BW_ACT_SILU, BW_ACT_CLAMPED_SWISH with its limit and alpha, BW_ACT_GELU_TANH)
BW_EXPORT int bw_glu(const void* gu, int in_type, void* out, int out_type, int T, int I, int act, float limit, float alpha,
                     void* stream) {
    if (act != BW_ACT_SILU && act != BW_ACT_CLAMPED_SWISH && act != BW_ACT_GELU_TANH) return BW_ERR_BAD_ARG;
    return launch_glu(gu, in_type, out, out_type, T, I, act, limit, alpha, stream);
}

// out[i] = act(x[i]) over n elements; act: BW_ACT_RELU2
BW_EXPORT int bw_unary_act(const void* x, int in_type, void* out, int out_type, long long n, int act, void* stream) {
    if (n <= 0) return 0;
    if (act != BW_ACT_RELU2) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    if (in_type == BW_F32 && out_type == BW_F32) bw::launch((unary_act_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, cp<float>(x), mp<float>(out), (size_t)n, act);
    else if (in_type == BW_BF16 && out_type == BW_BF16) bw::launch((unary_act_kernel<bf16, bf16>), dim3(blocks), dim3(threads), 0, s, cp<bf16>(x), mp<bf16>(out), (size_t)n, act);
    else if (in_type == BW_F32 && out_type == BW_BF16) bw::launch((unary_act_kernel<float, bf16>), dim3(blocks), dim3(threads), 0, s, cp<float>(x), mp<bf16>(out), (size_t)n, act);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// o [T, nh, dpad] of o_type, in place; g float32 [T, >= nh * dv] with rows ld floats apart
BW_EXPORT int bw_sigmoid_gate(void* o, int o_type, const float* g, long long ld, int T, int nh, int dv, int dpad, void* stream) {
    if (T <= 0) return 0;
    if (nh <= 0 || dv <= 0 || dpad < dv || ld < (long long)nh * dv) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (o_type == BW_F32) bw::launch((sigmoid_gate_kernel<float>), dim3(T), dim3(256), 0, s, mp<float>(o), g, ld, nh, dv, dpad);
    else if (o_type == BW_BF16) bw::launch((sigmoid_gate_kernel<bf16>), dim3(T), dim3(256), 0, s, mp<bf16>(o), g, ld, nh, dv, dpad);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

static int launch_glu(const void* gu, int in_type, void* out, int out_type, int T, int I, int act, float limit, float alpha, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (in_type == BW_F32 && out_type == BW_F32) bw::launch((swiglu_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, cp<float>(gu), mp<float>(out), I, total, act, limit, alpha);
    else if (in_type == BW_BF16 && out_type == BW_BF16) bw::launch((swiglu_kernel<bf16, bf16>), dim3(blocks), dim3(threads), 0, s, cp<bf16>(gu), mp<bf16>(out), I, total, act, limit, alpha);
    else if (in_type == BW_F32 && out_type == BW_BF16) bw::launch((swiglu_kernel<float, bf16>), dim3(blocks), dim3(threads), 0, s, cp<float>(gu), mp<bf16>(out), I, total, act, limit, alpha);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// magnitude: a factor on every cosine and sine (1 for plain rotary encoding; frequency rescalings that
// lengthen the context may ask for another)
BW_EXPORT int bw_rope_table(const int* positions, const float* inv_freq, float* table, int rotary_dim, int T,
                            float magnitude, void* stream) {
    if (T <= 0 || rotary_dim <= 0) return 0;
    if (rotary_dim & 1) return BW_ERR_BAD_ARG;
    const int total = T * (rotary_dim / 2);
    bw::launch((rope_table_kernel), dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, positions, inv_freq, table, rotary_dim, T, magnitude);
    BW_LAUNCH_CHECK();
    return 0;
}

BW_EXPORT int bw_kv_slots(const int* positions, const int* req_of_token, const int* block_table, int max_blocks,
                          int page_size, int num_pages, int* kv_slot, int T, void* stream) {
    if (T <= 0) return 0;
    if (page_size <= 0 || (long long)num_pages * page_size > 2147483647LL) return BW_ERR_BAD_ARG;
    bw::launch((kv_slots_kernel), dim3((T + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, req_of_token,
               block_table, max_blocks, page_size, num_pages, kv_slot, T);
    BW_LAUNCH_CHECK();
    return 0;
}

// table: [T, rotary_dim] from bw_rope_table, or null to compute the angles here.  paired != 0: the
// rotated channels of the q and k heads come as (channel j, channel j + rotary_dim / 2) pairs.
// n_planes > 1: qkv is the sum of that many planes, plane_stride elements apart (bw_gemm_tc_planes).
BW_EXPORT int bw_rope_append(const void* qkv, int in_type, const int* positions, const int* req_of_token,
                             const int* block_table, int max_blocks, const float* inv_freq, const float* table,
                             int rotary_dim, void* q_out, void* k_pages, void* v_pages, int out_type,
                             int T, int nh, int nkv, int hd, int page_size, int num_pages, int paired,
                             int n_planes, long long plane_stride, void* stream) {
    if (T <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) || n_planes < 1 || (n_planes > 1 && plane_stride <= 0)) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hd >= 256 ? 256 : (hd >= 128 ? 128 : (hd >= 64 ? 64 : 32));
    const dim3 grid(T, (nh + 2 * nkv + ROPE_HPB - 1) / ROPE_HPB);
#define BW_RA(IT, OT) bw::launch((rope_append_kernel<IT, OT>), dim3(grid), dim3(threads), 0, s, cp<IT>(qkv), positions, req_of_token, \
        block_table, max_blocks, inv_freq, table, rotary_dim, mp<OT>(q_out), mp<OT>(k_pages), mp<OT>(v_pages), \
        nh, nkv, hd, page_size, num_pages, paired, n_planes, (size_t)plane_stride)
    if (in_type == BW_F32 && out_type == BW_F32) BW_RA(float, float);
    else if (in_type == BW_F32 && out_type == BW_BF16) BW_RA(float, bf16);
    else if (in_type == BW_BF16 && out_type == BW_BF16) BW_RA(bf16, bf16);
    else return BW_ERR_BAD_ARG;
#undef BW_RA
    BW_LAUNCH_CHECK();
    return 0;
}
