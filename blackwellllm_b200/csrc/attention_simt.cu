// Paged causal grouped-query attention on the CUDA cores, all arithmetic float32.
// This is the attention of the true 32-bit path, and the plain twin that the
// tensor-core attention kernel is tested against.  One block (4 warps) per
// (token, query head); it takes any mix of prompt portions and decode tokens,
// because every token carries its own position and request.
//
// Keys are visited in 32-key chunks; chunk i belongs to warp i % 4, and the four
// partial results are merged in warp order.  The order of the sums is therefore a
// function of the key positions alone, never of the batch.
#include "common.cuh"

using bf16 = __nv_bfloat16;

namespace {

constexpr int WARPS = 4;
constexpr int HD_LIMIT = 1024;   // the kernel is built for 8 channels a lane (head sizes up to 256) and for 32 (up to 1024)

template <typename QT, typename KT, typename OT, int MAX_CH>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const QT* __restrict__ q, const KT* __restrict__ k_pages,
                      const KT* __restrict__ v_pages, const int* __restrict__ positions,
                      const int* __restrict__ req_of_token, const int* __restrict__ block_table,
                      int max_blocks, OT* __restrict__ out, int nh, int nkv, int hd, int page_size,
                      int num_pages, int window, int chunk, float scale, const float* __restrict__ sink,
                      const float* __restrict__ gate, long long gate_ld, int gate_dv,
                      const float* __restrict__ dist, int keep_first, float softcap, const float* __restrict__ rel,
                      int rel_len) {
    extern __shared__ float smem[];
    float* qs = smem;                       // [hd]
    float* accs = qs + hd;                  // [WARPS][hd]
    float* ml = accs + WARPS * hd;          // [WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / (nh / nkv);
    const int q_pos = positions[t];
    const int r = req_of_token[t];
    const int* bt = block_table + (size_t)r * max_blocks;
    const int lo = bw::first_visible(q_pos, window, chunk);
    // the keys a row walks: the kept first keys that lie before the window, then the window's
    const int n_kept = keep_first < lo ? (keep_first > 0 ? keep_first : 0) : lo;
    const int n_keys = n_kept + q_pos - lo + 1;
    const float r1 = dist ? dist[h] : 0.f, r2 = dist ? dist[nh + h] : 0.f;

    for (int c = threadIdx.x; c < hd; c += blockDim.x)
        qs[c] = bw::to_f32(q[((size_t)t * nh + h) * hd + c]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[MAX_CH];
#pragma unroll
    for (int i = 0; i < MAX_CH; ++i) acc[i] = 0.f;

    const int n_chunks = (n_keys + 31) / 32;
    for (int ch = warp; ch < n_chunks; ch += WARPS) {
        const int kn = ch * 32 + lane;               // this lane's key, counted along the row's walk
        const int kp = kn < n_kept ? kn : lo + (kn - n_kept);
        const bool valid = kp <= q_pos;
        float s = -INFINITY;
        size_t row_off = 0;
        if (valid) {
            const int page = bt[kp / page_size];
            if (page >= 0 && page < num_pages) {
                row_off = (((size_t)page * nkv + kvh) * page_size + (kp % page_size)) * hd;
                const KT* kr = k_pages + row_off;
                float d = 0.f;
                for (int c = 0; c < hd; ++c) d = fmaf(qs[c], bw::to_f32(kr[c]), d);
                s = d * scale;
                if (softcap > 0.f) s = bw::soft_cap(s, softcap);
                if (dist) s -= bw::distance_bias(r1, r2, q_pos - kp);
                if (rel) s += bw::table_bias(rel + (size_t)h * rel_len, rel_len, q_pos - kp);
            }
        }
        const float cm = bw::warp_max(s);
        const float m_new = fmaxf(m, cm);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        l = l * corr + bw::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < MAX_CH; ++i) acc[i] *= corr;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const size_t off = (size_t)__shfl_sync(0xffffffffu, (unsigned long long)row_off, j);
            if (pj == 0.f) continue;   // masked or beyond the last key (uniform across the warp)
            const KT* vr = v_pages + off;
#pragma unroll
            for (int i = 0; i < MAX_CH; ++i) {
                const int c = lane + 32 * i;
                if (c < hd) acc[i] = fmaf(pj, bw::to_f32(vr[c]), acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) accs[warp * hd + c] = acc[i];
    }
    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = l; }
    __syncthreads();
    // merge the warps' partial softmaxes in warp order
    float M = -INFINITY;
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, ml[w * 2]);
    float L = 0.f;
    float f[WARPS];
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (ml[w * 2] == -INFINITY) ? 0.f : expf(ml[w * 2] - M);
        L += ml[w * 2 + 1] * f[w];
    }
    if (sink) L += expf(sink[h] - M);   // one more term of the softmax, without a key or a value
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = threadIdx.x; c < hd; c += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; ++w) o += accs[w * hd + c] * f[w];
        out[((size_t)t * nh + h) * hd + c] = bw::from_f32<OT>(o * inv * bw::out_gate(gate, gate_ld, gate_dv, (size_t)t, h, c));
    }
}

}  // namespace

// sink: float32 [nh] or null: exp(sink[head]) joins every row's softmax denominator (unscaled, no key, no value).
// gate: float32 [T, >= nh * gate_dv], rows gate_ld apart, or null: output channel c < gate_dv of (token, head) is
// multiplied by sigmoid(gate[token, head * gate_dv + c]); channels from gate_dv on become zero.
// type: element type of q, the pages and out (all the same).  window <= 0: no window; chunk <= 0: no blocks (bw::first_visible).
// dist: float32 [2, nh] (r1 of every head, then r2) or null: r1 ln(1 + r2 (query position - key position)) is taken off
// every score.  keep_first: the first so many keys of a sequence stay visible whatever the window says.  gate_dv < 0:
// one gate number per head (bw::out_gate).  softcap > 0: the scaled score s becomes softcap * tanh(s / softcap) before any
// bias.  rel: float32 [nh][rel_len] or null: rel[head][min(query position - key position, rel_len - 1)] is added to the score.
BW_EXPORT int bw_attention_simt(const void* q, const void* k_pages, const void* v_pages, int type,
                                const int* positions, const int* req_of_token, const int* block_table,
                                int max_blocks, void* out, int T, int nh, int nkv, int hd, int page_size,
                                int num_pages, int window, int chunk, float scale, const float* sink, const float* gate,
                                long long gate_ld, int gate_dv, const float* dist, int keep_first, float softcap,
                                const float* rel, int rel_len, void* stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > HD_LIMIT || nkv <= 0 || nh % nkv != 0) return BW_ERR_UNSUPPORTED;
    if (rel && rel_len <= 0) return BW_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, nh);
    const size_t smem = (size_t)(hd + WARPS * hd + WARPS * 2) * sizeof(float);
#define BW_SIMT(TY, CH) attention_simt_kernel<TY, TY, TY, CH><<<grid, WARPS * 32, smem, s>>>( \
        (const TY*)q, (const TY*)k_pages, (const TY*)v_pages, positions, req_of_token, block_table, max_blocks, (TY*)out, nh, \
        nkv, hd, page_size, num_pages, window, chunk, scale, sink, gate, gate_ld, gate_dv, dist, keep_first, softcap, rel, rel_len)
    if (type == BW_F32) { if (hd <= 256) BW_SIMT(float, 8); else BW_SIMT(float, 32); }
    else if (type == BW_BF16) { if (hd <= 256) BW_SIMT(bf16, 8); else BW_SIMT(bf16, 32); }
#undef BW_SIMT
    else return BW_ERR_BAD_ARG;
    BW_LAUNCH_CHECK();
    return 0;
}
