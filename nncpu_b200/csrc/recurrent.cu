// Recurrent mixers: layers that carry a fixed-size state per sequence from token to token instead of keys
// and values per position.  The state lives in 32-bit floats in the cache's state area, one row per sequence
// slot; everything that enters the recurrence (decays, their logarithms and exponentials) is computed in 32-bit.
//
// Gated linear attention.  Per head, with a state S of d rows (key channels) and e columns (value channels):
//     a_t = sigmoid(z_t)^(1/tau)                 (a decay per key channel, from the gate logits z_t)
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T
//     o_t = S_t^T q_t
// The columns of S do not depend on one another, so a warp owns 32 of them (a lane one column, its d
// numbers in registers) and walks the tokens of its sequence in order; q, k and a of a token are shared by
// the warp through shared memory.  The order of operations of a (sequence, head, column) does not depend on
// how the sequence was cut into steps or on what else the step holds, so the results are the same bits.

#include <math.h>

#define NN_LIB recurrent
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// proj [n_tok, row] float32 holds per token q (H*d), k (H*d), v (H*e), g (H*e); z [n_tok, H*d] float32 the
// decay logits.  state [n_slots + 1, H, d, e]; seq_slots[s] < 0 marks a padding sequence: its rows of o are zero
// and no state is touched.  o [n_tok, H*e] float32.
template <int DMAX>
__global__ void __launch_bounds__(32)
gla_scan_kernel(const float* __restrict__ proj, int row, const float* __restrict__ z, float* __restrict__ state,
                const int* __restrict__ seq_slots, const int* __restrict__ cu_seqlens, float* __restrict__ o, int H,
                int d, int e, float q_scale, float inv_tau) {
    constexpr int PER = DMAX / 32;              // key channels a lane fetches per token
    __shared__ float4 shared[DMAX];             // (a, k, q, -) of the token under way
    const int seq = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int j = blockIdx.z * 32 + lane;
    const bool live = j < e;
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const int slot = seq_slots[seq];
    if (slot < 0) {
        if (live)
            for (int t = t0; t < t1; ++t) o[(size_t)t * H * e + (size_t)h * e + j] = 0.0f;
        return;
    }
    float* s_col = state + (((size_t)slot * H + h) * d) * e + j;
    float S[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = (live && i < d) ? s_col[(size_t)i * e] : 0.0f;

    const size_t q_at = (size_t)h * d, k_at = (size_t)H * d + (size_t)h * d, v_at = 2 * (size_t)H * d + (size_t)h * e;
    float nq[PER], nk[PER], nz[PER], nv = 0.0f;
    auto fetch = [&](int t) {
        const float* p = proj + (size_t)t * row;
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int i = lane + 32 * c;
            if (i < d) {
                nq[c] = p[q_at + i];
                nk[c] = p[k_at + i];
                nz[c] = z[(size_t)t * H * d + (size_t)h * d + i];
            }
        }
        nv = live ? p[v_at + j] : 0.0f;
    };
    if (t0 < t1) fetch(t0);
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int i = lane + 32 * c;
            if (i < d) shared[i] = make_float4(expf(log_sigmoid_f(nz[c]) * inv_tau), nk[c], nq[c] * q_scale, 0.0f);
        }
        const float v = nv;
        __syncwarp();
        if (t + 1 < t1) fetch(t + 1);           // the next token's loads fly under this token's arithmetic
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < DMAX; ++i) {
            if (i < d) {
                const float4 c = shared[i];
                S[i] = fmaf(c.x, S[i], c.y * v);
                acc = fmaf(S[i], c.z, acc);
            }
        }
        if (live) o[(size_t)t * H * e + (size_t)h * e + j] = acc;
        __syncwarp();
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i < d) s_col[(size_t)i * e] = S[i];
    }
}

extern "C" int nncpu_gla_scan(const float* proj, int row, const float* z, float* state, const int* seq_slots,
                              const int* cu_seqlens, float* o, int n_seqs, int H, int d, int e, float q_scale,
                              float tau, void* stream) {
    NN_CHECK(n_seqs >= 0 && H > 0 && d > 0 && e > 0, "gla_scan: %d sequences, %d heads of %d x %d", n_seqs, H, d, e);
    NN_CHECK(d <= 256, "gla_scan: %d key channels a head (at most 256)", d);
    NN_CHECK(row >= 2 * H * d + 2 * H * e, "gla_scan: rows of %d floats for %d heads of %d x %d", row, H, d, e);
    NN_CHECK(tau > 0.0f, "gla_scan: tau %g", tau);
    NN_CHECK(H <= 65535 && (e + 31) / 32 <= 65535, "gla_scan: grid");
    if (n_seqs == 0) return 0;
    dim3 grid(n_seqs, H, (e + 31) / 32);
    const float inv_tau = 1.0f / tau;
    cudaStream_t st = (cudaStream_t)stream;
    if (d <= 32) gla_scan_kernel<32><<<grid, 32, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, e, q_scale, inv_tau);
    else if (d <= 64) gla_scan_kernel<64><<<grid, 32, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, e, q_scale, inv_tau);
    else if (d <= 128) gla_scan_kernel<128><<<grid, 32, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, e, q_scale, inv_tau);
    else gla_scan_kernel<256><<<grid, 32, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, e, q_scale, inv_tau);
    NN_LAUNCH_OK("gla_scan");
    return 0;
}

// The mixer's output stage: every head's o is divided by its root mean square over the e value channels (eps
// inside the root), multiplied by the weight w [e] that the heads share and by silu(g), the gate of its channel.
// One warp per (token, head); out [n_tok, H*e] in the run's element type.
__global__ void __launch_bounds__(256)
gla_output_kernel(const float* __restrict__ o, const float* __restrict__ proj, int row, int g_at,
                  const void* __restrict__ w, int w_dt, float eps, void* __restrict__ out, int out_dt, long n_items,
                  int H, int e) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= n_items) return;
    const long t = item / H;
    const int h = (int)(item % H);
    const float* src = o + (size_t)t * H * e + (size_t)h * e;
    float ss = 0.0f;
    for (int j = lane; j < e; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss * (1.0f / (float)e) + eps);
    const float* g = proj + (size_t)t * row + g_at + (size_t)h * e;
    for (int j = lane; j < e; j += 32) {
        const float gate = g[j];
        const float y = (src[j] * scale) * ld_f(w, j, w_dt);
        st_f(out, (size_t)t * H * e + (size_t)h * e + j, out_dt, y * (gate / (1.0f + expf(-gate))));
    }
}

extern "C" int nncpu_gla_output(const float* o, const float* proj, int row, int g_at, const void* w, int w_dt,
                                float eps, void* out, int out_dt, int n_tok, int H, int e, void* stream) {
    NN_CHECK(n_tok >= 0 && H > 0 && e > 0 && g_at >= 0 && g_at + H * e <= row, "gla_output: sizes");
    if (n_tok == 0) return 0;
    const long n_items = (long)n_tok * H;
    gla_output_kernel<<<(unsigned)((n_items + 7) / 8), 256, 0, (cudaStream_t)stream>>>(o, proj, row, g_at, w, w_dt, eps,
                                                                                       out, out_dt, n_items, H, e);
    NN_LAUNCH_OK("gla_output");
    return 0;
}
