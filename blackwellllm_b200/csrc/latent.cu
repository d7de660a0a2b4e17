// Kernels of the latent-attention mixer: keys and values of all heads are made from one small latent vector c per
// token, and only c and one rotated key part shared by the heads are cached.  The heads' key and value matrices
// are moved to the query's and the output's side ("absorbed"), so that the attention itself is a grouped-query
// attention with ONE key/value head whose key row is [c, rotated part] and whose value row is c:
//     score_h(i, j) = (W_uk,h^T q_plain,h(i)) . c(j) + q_rot,h(i) . k_rot(j)        out_h(i) = W_uv,h (sum_j p_ij c(j))
//   * latent_prep: RMS norm of the latent with its gain, rotation of the shared key part and of the queries' rotated
//     parts, append of [c, k_rot, 0...] to the token's cache row;
//   * headwise_linear: y[t, h, :] = W[h] x[t, h, :] for every head h (a small product per head: W_uk,h^T on the queries,
//     W_uv,h on the attention's output), float32 sums in a fixed order: on the CUDA cores in float32, on the tensor
//     cores (mma.sync) with bfloat16 weights.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

template <typename OT>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const float* __restrict__ qsrc, long long q_ld, int q_off, const float* __restrict__ proj, long long ld,
                   int kv_off, int interleaved, const int* __restrict__ positions,
                   const int* __restrict__ req_of_token, const int* __restrict__ block_table, int max_blocks,
                   const float* __restrict__ table, const float* __restrict__ c_gain, float eps, OT* __restrict__ q_out,
                   OT* __restrict__ k_pages, int H, int d, int dr, int rank, int dpad, int page_size, int num_pages) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const float* qrow = qsrc + (size_t)t * q_ld;
    const float* tab = table + (size_t)t * dr;     // cosines, then sines (both already times the magnitude)
    const int half = dr >> 1;
    // channel c turns with channel c + dr / 2 (pair c mod dr / 2), or, interleaved, channel 2j with channel 2j + 1 (pair j)
    auto turned = [&](const float* src, int c) {
        const bool first = interleaved ? !(c & 1) : c < half;
        const int j = interleaved ? c >> 1 : (first ? c : c - half);
        const int pc = interleaved ? c ^ 1 : (first ? c + half : c - half);
        const float x = src[c], y = src[pc];
        return first ? x * tab[j] - y * tab[half + j] : x * tab[j] + y * tab[half + j];
    };
    // the queries' rotated parts, behind the room for the absorbed plain parts; pad channels zero
    const int tail = dpad - rank;
    for (int idx = threadIdx.x; idx < H * tail; idx += blockDim.x) {
        const int h = idx / tail, c = idx - h * tail;
        const float o = c < dr ? turned(qrow + q_off + (size_t)h * (d + dr) + d, c) : 0.f;
        q_out[((size_t)t * H + h) * dpad + rank + c] = bw::from_f32<OT>(o);
    }
    if (num_pages <= 0) return;
    const int pos = positions[t];
    int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) return;     // (uniform over the block)
    const float* kv = row + kv_off;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float v = kv[c]; ss = fmaf(v, v, ss); }
    const float r = rsqrtf(bw::block_sum(ss, scratch) / (float)rank + eps);
    OT* dst = k_pages + ((size_t)page * page_size + pos % page_size) * dpad;
    for (int c = threadIdx.x; c < dpad; c += blockDim.x) {
        float o = 0.f;
        if (c < rank) o = kv[c] * r * c_gain[c];
        else if (c < rank + dr) o = turned(kv + rank, c - rank);
        dst[c] = bw::from_f32<OT>(o);
    }
}

// An output gate on a per-head product's result: sigmoid(gate[t, h * n_out + o]) (float32 rows g_ld apart), 1 without a gate.
__device__ __forceinline__ float head_gate(const float* __restrict__ gate, long long g_ld, int t, int h, int n_out, int o) {
    return gate ? 1.f / (1.f + expf(-gate[(size_t)t * g_ld + (size_t)h * n_out + o])) : 1.f;
}

// y[t, h * y_hs + o] = sum_i x[t, h * x_hs + i] * w[h, o, i]:  tiles of 32 tokens x 64 outputs, 32 inner values at a time.
constexpr int HT = 32, HO = 64, HK = 32;
template <typename XT, typename WT, typename YT>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const XT* __restrict__ x, long long ldx, int x_hs, const WT* __restrict__ w, YT* __restrict__ y,
                       long long ldy, int y_hs, int T, int n_in, int n_out, const float* __restrict__ gate, long long g_ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float xs[HT][HK + 1];
    __shared__ float ws[HO][HK + 1];
    const int h = blockIdx.z, t0 = blockIdx.x * HT, o0 = blockIdx.y * HO;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // 16 x 16: four outputs and two tokens a thread
    const WT* wh = w + (size_t)h * n_out * n_in;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int k0 = 0; k0 < n_in; k0 += HK) {
        for (int idx = threadIdx.x; idx < HT * HK; idx += 256) {
            const int r = idx / HK, k = idx - r * HK;
            const int t = t0 + r, i = k0 + k;
            xs[r][k] = (t < T && i < n_in) ? bw::to_f32(x[(size_t)t * ldx + (size_t)h * x_hs + i]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < HO * HK; idx += 256) {
            const int r = idx / HK, k = idx - r * HK;
            const int o = o0 + r, i = k0 + k;
            ws[r][k] = (o < n_out && i < n_in) ? bw::to_f32(wh[(size_t)o * n_in + i]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < HK; ++k) {
            const float a0 = xs[ty * 2][k], a1 = xs[ty * 2 + 1][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = ws[tx + 16 * j][k];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int t = t0 + ty * 2 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o < n_out) y[(size_t)t * ldy + (size_t)h * y_hs + o] = bw::from_f32<YT>(acc[i][j] * head_gate(gate, g_ld, t, h, n_out, o));
        }
    }
}

// The same product on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums) for bfloat16 weights and
// results: a CTA of 4 warps makes 64 tokens x 64 outputs of one head, warp w the tokens 16 w .. 16 w + 15; the operands
// pass through shared memory 64 inner values at a time (float32 inputs are rounded to bfloat16 on the way; 16-byte
// loads where sizes and addresses allow them: `vec`), rows padded to 144 bytes so that the 8 rows of an ldmatrix fall into different banks.
constexpr int MT = 64, MO = 64, MK = 64, MROW = (MK + 8) * 2;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename XT>
__global__ void __launch_bounds__(128)
headwise_mma_kernel(const XT* __restrict__ x, long long ldx, int x_hs, const bf16* __restrict__ w, bf16* __restrict__ y,
                    long long ldy, int y_hs, int T, int n_in, int n_out, int vec, const float* __restrict__ gate, long long g_ld) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ __align__(16) uint8_t xs[MT * MROW];
    __shared__ __align__(16) uint8_t ws[MO * MROW];
    const int h = blockIdx.z, t0 = blockIdx.x * MT, o0 = blockIdx.y * MO;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bf16* wh = w + (size_t)h * n_out * n_in;
    float acc[MO / 8][4];
#pragma unroll
    for (int j = 0; j < MO / 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
    // every thread stages 32 inner values of one row of each operand, 8 at a time
    const int srow = threadIdx.x >> 1, scol = (threadIdx.x & 1) * 32;
    for (int k0 = 0; k0 < n_in; k0 += MK) {
        const int t = t0 + srow, o = o0 + srow;
        const XT* src = x + (size_t)(t < T ? t : 0) * ldx + (size_t)h * x_hs + k0 + scol;
        const bf16* wsrc = wh + (size_t)(o < n_out ? o : 0) * n_in + k0 + scol;
        uint8_t* dst = xs + srow * MROW + scol * 2;
        uint8_t* wdst = ws + srow * MROW + scol * 2;
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
            const bool in = k0 + scol + c < n_in;      // (vec: n_in is a multiple of 8, so a chunk is inside or outside)
            uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
            if (vec) {
                if (in && t < T) {
                    if constexpr (sizeof(XT) == 4) {
                        const float4 lo = *reinterpret_cast<const float4*>(src + c), hi = *reinterpret_cast<const float4*>(src + c + 4);
                        xv = make_uint4(bw::pack_bf16x2(lo.x, lo.y), bw::pack_bf16x2(lo.z, lo.w), bw::pack_bf16x2(hi.x, hi.y), bw::pack_bf16x2(hi.z, hi.w));
                    } else {
                        xv = *reinterpret_cast<const uint4*>(src + c);
                    }
                }
                if (in && o < n_out) wv = __ldg(reinterpret_cast<const uint4*>(wsrc + c));
            } else {
                bf16 xe[8], we[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool ok = k0 + scol + c + i < n_in;
                    xe[i] = (ok && t < T) ? bw::from_f32<bf16>(bw::to_f32(src[c + i])) : __float2bfloat16_rn(0.f);
                    we[i] = (ok && o < n_out) ? wsrc[c + i] : __float2bfloat16_rn(0.f);
                }
                xv = *reinterpret_cast<const uint4*>(xe);
                wv = *reinterpret_cast<const uint4*>(we);
            }
            *reinterpret_cast<uint4*>(dst + c * 2) = xv;
            *reinterpret_cast<uint4*>(wdst + c * 2) = wv;
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < MK / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(smem_addr(xs) + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * MROW + 16 * (lane >> 4) + ks * 32,
                    a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int nb = 0; nb < MO / 16; ++nb) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_addr(ws) + (nb * 16 + (lane & 7) + 8 * (lane >> 4)) * MROW + 16 * ((lane >> 3) & 1) + ks * 32, b0, b1, b2, b3);
                mma_bf16(acc[2 * nb], a, b0, b1);
                mma_bf16(acc[2 * nb + 1], a, b2, b3);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int t = t0 + warp * 16 + (lane >> 2) + 8 * half;
        if (t >= T) continue;
        bf16* dst = y + (size_t)t * ldy + (size_t)h * y_hs;
        const bool pairs = ((reinterpret_cast<uintptr_t>(dst) & 3) == 0);   // (o is even: a pair of results is one 4-byte store)
#pragma unroll
        for (int j = 0; j < MO / 8; ++j) {
            const int o = o0 + j * 8 + 2 * (lane & 3);
            float r0 = acc[j][2 * half], r1 = acc[j][2 * half + 1];
            if (gate) {
                if (o < n_out) r0 *= head_gate(gate, g_ld, t, h, n_out, o);
                if (o + 1 < n_out) r1 *= head_gate(gate, g_ld, t, h, n_out, o + 1);
            }
            if (pairs && o + 1 < n_out) {
                *reinterpret_cast<uint32_t*>(dst + o) = bw::pack_bf16x2(r0, r1);
            } else {
                if (o < n_out) dst[o] = __float2bfloat16_rn(r0);
                if (o + 1 < n_out) dst[o + 1] = __float2bfloat16_rn(r1);
            }
        }
    }
}

}  // namespace

// proj: float32 rows `ld` apart; queries at column q_off, H heads of (d plain, dr rotated) channels; the latent's
// projection at column kv_off: rank channels, then the dr channels of the shared key part.  table float32 [T, dr].
// q_out [T, H, dpad] and the pages [num_pages, 1, page_size, dpad] of out_type, dpad >= rank + dr.  Channels
// [0, rank) of q_out are left for headwise_linear.  num_pages <= 0: nothing is appended.
// qsrc: the queries' rows (float32, q_ld apart, H heads of d + dr channels from column q_off on); proj: the rows that hold
// the latent and the shared key part at column kv_off (the same tensor as qsrc, or another).  interleaved != 0: the rotation
// pairs channel 2j with channel 2j + 1 instead of channel c with channel c + dr / 2.
BW_EXPORT int bw_latent_prep(const float* qsrc, long long q_ld, int q_off, const float* proj, long long ld, int kv_off,
                             int interleaved, const int* positions,
                             const int* req_of_token, const int* block_table, int max_blocks, const float* table,
                             const float* c_gain, float eps, void* q_out, void* k_pages, int out_type, int T, int H, int d,
                             int dr, int rank, int dpad, int page_size, int num_pages, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0 || dr <= 0 || (dr & 1) || rank <= 0 || dpad < rank + dr || page_size <= 0 || !table || !c_gain ||
        !qsrc || !proj || q_ld < (long long)q_off + (long long)H * (d + dr) || ld < (long long)kv_off + rank + dr)
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32)
        bw::launch((latent_prep_kernel<float>), dim3(T), dim3(256), 0, s, qsrc, q_ld, q_off, proj, ld, kv_off, interleaved,
                   positions, req_of_token,
                   block_table, max_blocks, table, c_gain, eps, (float*)q_out, (float*)k_pages, H, d, dr, rank, dpad,
                   page_size, num_pages);
    else if (out_type == BW_BF16)
        bw::launch((latent_prep_kernel<bf16>), dim3(T), dim3(256), 0, s, qsrc, q_ld, q_off, proj, ld, kv_off, interleaved,
                   positions, req_of_token,
                   block_table, max_blocks, table, c_gain, eps, (bf16*)q_out, (bf16*)k_pages, H, d, dr, rank, dpad,
                   page_size, num_pages);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// x: rows ldx apart, head h's n_in inputs at column h * x_hs; w [H, n_out, n_in]; y: rows ldy apart, head h's n_out
// outputs at column h * y_hs.  Types: x float32 or bfloat16; w and y float32 or bfloat16 (the same for both).
// gate: null, or float32 rows g_ld apart with H * n_out values: the result is multiplied by sigmoid(gate[t, h * n_out + o])
// before it is rounded and written.
BW_EXPORT int bw_headwise_linear(const void* x, int x_type, long long ldx, int x_hs, const void* w, int w_type, void* y,
                                 int y_type, long long ldy, int y_hs, int T, int H, int n_in, int n_out, const float* gate,
                                 long long g_ld, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || n_in <= 0 || n_out <= 0 || H > 65535 || (gate && g_ld < (long long)H * n_out)) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((T + HT - 1) / HT, (n_out + HO - 1) / HO, H);
#define BW_HW(XT, WT, YT) bw::launch((headwise_linear_kernel<XT, WT, YT>), grid, dim3(256), 0, s, (const XT*)x, ldx, x_hs, \
        (const WT*)w, (YT*)y, ldy, y_hs, T, n_in, n_out, gate, g_ld)
    const dim3 mgrid((T + MT - 1) / MT, (n_out + MO - 1) / MO, H);
    // 16-byte loads: 8 inner values of a row at a time, every row starting on a 16-byte boundary
    const int xe = x_type == BW_F32 ? 4 : 8;      // elements of x in 16 bytes
    const int vec = n_in % 8 == 0 && ldx % xe == 0 && x_hs % xe == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
    if (x_type == BW_F32 && w_type == BW_F32 && y_type == BW_F32) BW_HW(float, float, float);
    else if (x_type == BW_F32 && w_type == BW_BF16 && y_type == BW_BF16)      // bfloat16 weights and results: the tensor cores
        bw::launch((headwise_mma_kernel<float>), mgrid, dim3(128), 0, s, (const float*)x, ldx, x_hs, (const bf16*)w, (bf16*)y, ldy, y_hs, T, n_in, n_out, vec, gate, g_ld);
    else if (x_type == BW_BF16 && w_type == BW_BF16 && y_type == BW_BF16)
        bw::launch((headwise_mma_kernel<bf16>), mgrid, dim3(128), 0, s, (const bf16*)x, ldx, x_hs, (const bf16*)w, (bf16*)y, ldy, y_hs, T, n_in, n_out, vec, gate, g_ld);
    else return BW_ERR_UNSUPPORTED;
#undef BW_HW
    BW_LAUNCH_CHECK();
    return 0;
}
