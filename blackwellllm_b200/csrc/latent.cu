// Kernels of the latent-attention mixer: keys and values of all heads are made from one small latent vector c per
// token, and only c and one rotated key part shared by the heads are cached.  The heads' key and value matrices
// are moved to the query's and the output's side ("absorbed"), so that the attention itself is a grouped-query
// attention with ONE key/value head whose key row is [c, rotated part] and whose value row is c:
//     score_h(i, j) = (W_uk,h^T q_plain,h(i)) . c(j) + q_rot,h(i) . k_rot(j)        out_h(i) = W_uv,h (sum_j p_ij c(j))
//   * latent_prep: RMS norm of the latent with its gain, rotation of the shared key part and of the queries' rotated
//     parts, append of [c, k_rot, 0...] to the token's cache row;
//   * headwise_linear: y[t, h, :] = W[h] x[t, h, :] for every head h (a small product per head: W_uk,h^T on the queries,
//     W_uv,h on the attention's output), float32 sums in a fixed order.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

template <typename OT>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const float* __restrict__ proj, long long ld, int q_off, int kv_off, const int* __restrict__ positions,
                   const int* __restrict__ req_of_token, const int* __restrict__ block_table, int max_blocks,
                   const float* __restrict__ table, const float* __restrict__ c_gain, float eps, OT* __restrict__ q_out,
                   OT* __restrict__ k_pages, int H, int d, int dr, int rank, int dpad, int page_size, int num_pages) {
    BW_PDL_TRIGGER();
    BW_PDL_WAIT();
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const float* tab = table + (size_t)t * dr;     // cosines, then sines (both already times the magnitude)
    const int half = dr >> 1;
    auto turned = [&](const float* src, int c) {
        const bool first = c < half;
        const int j = first ? c : c - half;
        const float x = src[c], y = src[first ? c + half : c - half];
        return first ? x * tab[j] - y * tab[half + j] : x * tab[j] + y * tab[half + j];
    };
    // the queries' rotated parts, behind the room for the absorbed plain parts; pad channels zero
    const int tail = dpad - rank;
    for (int idx = threadIdx.x; idx < H * tail; idx += blockDim.x) {
        const int h = idx / tail, c = idx - h * tail;
        const float o = c < dr ? turned(row + q_off + (size_t)h * (d + dr) + d, c) : 0.f;
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

// y[t, h * y_hs + o] = sum_i x[t, h * x_hs + i] * w[h, o, i]:  tiles of 32 tokens x 64 outputs, 32 inner values at a time.
constexpr int HT = 32, HO = 64, HK = 32;
template <typename XT, typename WT, typename YT>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const XT* __restrict__ x, long long ldx, int x_hs, const WT* __restrict__ w, YT* __restrict__ y,
                       long long ldy, int y_hs, int T, int n_in, int n_out) {
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
            if (o < n_out) y[(size_t)t * ldy + (size_t)h * y_hs + o] = bw::from_f32<YT>(acc[i][j]);
        }
    }
}

}  // namespace

// proj: float32 rows `ld` apart; queries at column q_off, H heads of (d plain, dr rotated) channels; the latent's
// projection at column kv_off: rank channels, then the dr channels of the shared key part.  table float32 [T, dr].
// q_out [T, H, dpad] and the pages [num_pages, 1, page_size, dpad] of out_type, dpad >= rank + dr.  Channels
// [0, rank) of q_out are left for headwise_linear.  num_pages <= 0: nothing is appended.
BW_EXPORT int bw_latent_prep(const float* proj, long long ld, int q_off, int kv_off, const int* positions,
                             const int* req_of_token, const int* block_table, int max_blocks, const float* table,
                             const float* c_gain, float eps, void* q_out, void* k_pages, int out_type, int T, int H, int d,
                             int dr, int rank, int dpad, int page_size, int num_pages, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || d <= 0 || dr <= 0 || (dr & 1) || rank <= 0 || dpad < rank + dr || page_size <= 0 || !table || !c_gain ||
        ld < (long long)q_off + (long long)H * (d + dr) || ld < (long long)kv_off + rank + dr)
        return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_type == BW_F32)
        bw::launch((latent_prep_kernel<float>), dim3(T), dim3(256), 0, s, proj, ld, q_off, kv_off, positions, req_of_token,
                   block_table, max_blocks, table, c_gain, eps, (float*)q_out, (float*)k_pages, H, d, dr, rank, dpad,
                   page_size, num_pages);
    else if (out_type == BW_BF16)
        bw::launch((latent_prep_kernel<bf16>), dim3(T), dim3(256), 0, s, proj, ld, q_off, kv_off, positions, req_of_token,
                   block_table, max_blocks, table, c_gain, eps, (bf16*)q_out, (bf16*)k_pages, H, d, dr, rank, dpad,
                   page_size, num_pages);
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}

// x: rows ldx apart, head h's n_in inputs at column h * x_hs; w [H, n_out, n_in]; y: rows ldy apart, head h's n_out
// outputs at column h * y_hs.  Types: x float32 or bfloat16; w and y float32 or bfloat16 (the same for both).
BW_EXPORT int bw_headwise_linear(const void* x, int x_type, long long ldx, int x_hs, const void* w, int w_type, void* y,
                                 int y_type, long long ldy, int y_hs, int T, int H, int n_in, int n_out, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || n_in <= 0 || n_out <= 0 || H > 65535) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((T + HT - 1) / HT, (n_out + HO - 1) / HO, H);
#define BW_HW(XT, WT, YT) bw::launch((headwise_linear_kernel<XT, WT, YT>), grid, dim3(256), 0, s, (const XT*)x, ldx, x_hs, \
        (const WT*)w, (YT*)y, ldy, y_hs, T, n_in, n_out)
    if (x_type == BW_F32 && w_type == BW_F32 && y_type == BW_F32) BW_HW(float, float, float);
    else if (x_type == BW_F32 && w_type == BW_BF16 && y_type == BW_BF16) BW_HW(float, bf16, bf16);
    else if (x_type == BW_BF16 && w_type == BW_BF16 && y_type == BW_BF16) BW_HW(bf16, bf16, bf16);
    else return BW_ERR_UNSUPPORTED;
#undef BW_HW
    BW_LAUNCH_CHECK();
    return 0;
}
