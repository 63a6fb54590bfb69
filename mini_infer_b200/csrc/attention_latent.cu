// Row-wise kernels of attention through a latent: every token keeps ONE row [c + r] that all heads share, a
// latent of c numbers (divided by its root mean square, times a gain per dimension) from which each head's
// key and value are formed by matrices of the head, followed by r numbers of a key part that is rotated by
// position and common to all heads.  With the key matrices folded into the queries
// (q'_h = W_uk,h^T q_h, so that q_h . (W_uk,h c) = q'_h . c) the attention itself is the engine's attention
// over one shared key/value head whose keys are the cached rows and whose values are their first c numbers
// (attention_mix.cu and attention_mix_tc.cu with a value row stride, attention_prefill_tc.cu with (query, head)
// pairs as the rows of a query tile); what is left for this file:
//
//   latent_store   the cached row of every new token: unit-RMS latent times gain, rotated key part
//   latent_query   the rotated part of every head's query into its place behind the folded part, and the
//                  unrotated part in the activation type as the operand of the folding product
//   sigmoid_gate   out[t, h, :] = a[t, h, :] * sigmoid(g[t, h, :]), the gate on the heads' outputs
//
// The rotation pairs NEIGHBOURS: dimensions 2i and 2i + 1 turn by the angle position * inv_freq[i].  Angles,
// norms and the gate are float arithmetic in both precision paths.

#include "common.cuh"

namespace mi {

// one block per token; src row: `ld` floats, the latent part at column `col0`
template <typename AT>
__global__ void __launch_bounds__(256)
latent_store_kernel(const float* __restrict__ src, int ld, int col0, const int* __restrict__ positions,
                    const float* __restrict__ inv_freq, const float* __restrict__ gain, float eps,
                    const int* __restrict__ slot_mapping, AT* __restrict__ cache, int c, int r) {
    __shared__ float red[32];
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    const int slot = slot_mapping[t];
    if (slot < 0) return;                           // a row of no request: written nowhere
    const float* row = src + (int64_t)t * ld + col0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < c; i += blockDim.x) { const float x = row[i]; ss += x * x; }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)c + eps);
    AT* out = cache + (int64_t)slot * (c + r);
    for (int i = threadIdx.x; i < c; i += blockDim.x) out[i] = from_float<AT>(row[i] * inv * gain[i]);
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < r / 2; i += blockDim.x) {
        const float ang = pos * inv_freq[i];
        const float cs = cosf(ang), sn = sinf(ang);
        const float u = row[c + 2 * i], v = row[c + 2 * i + 1];
        out[c + 2 * i] = from_float<AT>(u * cs - v * sn);
        out[c + 2 * i + 1] = from_float<AT>(v * cs + u * sn);
    }
}

// one block per token; q row: H heads of [d unrotated | r rotated] floats
template <typename AT>
__global__ void __launch_bounds__(256)
latent_query_kernel(const float* __restrict__ q, const int* __restrict__ positions,
                    const float* __restrict__ inv_freq, AT* __restrict__ q_plain, AT* __restrict__ q_full, int H,
                    int d, int r, int c) {
    wait_for_earlier_kernels();
    const int t = blockIdx.x;
    const float* row = q + (int64_t)t * H * (d + r);
    const float pos = (float)positions[t];
    const int half = r / 2;
    for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const float ang = pos * inv_freq[i];
        const float cs = cosf(ang), sn = sinf(ang);
        const float u = row[h * (d + r) + d + 2 * i], v = row[h * (d + r) + d + 2 * i + 1];
        AT* out = q_full + ((int64_t)t * H + h) * (c + r) + c;
        out[2 * i] = from_float<AT>(u * cs - v * sn);
        out[2 * i + 1] = from_float<AT>(v * cs + u * sn);
    }
    if (q_plain)
        for (int idx = threadIdx.x; idx < H * d; idx += blockDim.x) {
            const int h = idx / d, i = idx - h * d;
            q_plain[(int64_t)t * H * d + idx] = from_float<AT>(row[h * (d + r) + i]);
        }
}

// out[t, h, j] = a[h * a_head + t * a_tok + j] * sigmoid(g[t * ldg + col0 + h * e + j])
template <typename AT>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const AT* __restrict__ a, int64_t a_head, int64_t a_tok, const float* __restrict__ g, int ldg,
                    int col0, AT* __restrict__ out, int T, int H, int e) {
    wait_for_earlier_kernels();
    const int64_t total = (int64_t)T * H * e;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(idx % e);
        const int h = (int)((idx / e) % H);
        const int64_t t = idx / ((int64_t)e * H);
        const float x = to_float(a[h * a_head + t * a_tok + j]);
        const float z = g[t * ldg + col0 + h * e + j];
        out[idx] = from_float<AT>(x / (1.0f + expf(-z)));
    }
}

// bfloat16 with e a multiple of 8 and 16-byte aligned rows: eight gated values per thread
__global__ void __launch_bounds__(256)
sigmoid_gate_bf16x8_kernel(const __nv_bfloat16* __restrict__ a, int64_t a_head, int64_t a_tok,
                           const float* __restrict__ g, int ldg, int col0, __nv_bfloat16* __restrict__ out, int T,
                           int H, int e8) {
    wait_for_earlier_kernels();
    const int64_t total = (int64_t)T * H * e8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(idx % e8) * 8;
        const int h = (int)((idx / e8) % H);
        const int64_t t = idx / ((int64_t)e8 * H);
        const uint4 av = __ldg(reinterpret_cast<const uint4*>(a + h * a_head + t * a_tok + j));
        const float4* gp = reinterpret_cast<const float4*>(g + t * ldg + col0 + h * (e8 * 8) + j);
        const float4 g0 = __ldg(gp), g1 = __ldg(gp + 1);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
        const float z[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x = __bfloat1622float2(ap[k]);
            op[k] = __floats2bfloat162_rn(x.x / (1.0f + expf(-z[2 * k])), x.y / (1.0f + expf(-z[2 * k + 1])));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

}  // namespace mi

using namespace mi;

extern "C" {

int mi_latent_store(const float* src, int ld, int col0, const int* positions, const float* inv_freq,
                    const float* gain, float eps, const int* slot_mapping, void* cache, int adtype, int T, int c,
                    int r, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (c < 1 || r < 0 || r % 2 || col0 < 0 || col0 + c + r > ld || (r > 0 && !inv_freq)) {
        set_last_error("latent_store: latent of %d and rotated part of %d at column %d of rows of %d", c, r, col0, ld);
        return kBadShape;
    }
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(latent_store_kernel<AT>, dim3(T), dim3(256), 0, stream, src, ld, col0, positions, inv_freq,
                         gain, eps, slot_mapping, (AT*)cache, c, r));
    return finish_launch("latent_store");
}

int mi_latent_query(const float* q, const int* positions, const float* inv_freq, void* q_plain, void* q_full,
                    int adtype, int T, int H, int d, int r, int c, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (H < 1 || d < 1 || r < 0 || r % 2 || c < 1 || (r > 0 && !inv_freq)) {
        set_last_error("latent_query: %d heads of %d + %d, latent of %d", H, d, r, c);
        return kBadShape;
    }
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(latent_query_kernel<AT>, dim3(T), dim3(256), 0, stream, q, positions, inv_freq,
                         (AT*)q_plain, (AT*)q_full, H, d, r, c));
    return finish_launch("latent_query");
}

int mi_sigmoid_gate(const void* a, int64_t a_head, int64_t a_tok, const float* g, int ldg, int col0, void* out,
                    int adtype, int T, int H, int e, cudaStream_t stream) {
    if (T <= 0) return kOk;
    if (H < 1 || e < 1 || col0 < 0 || col0 + H * e > ldg) {
        set_last_error("sigmoid_gate: %d heads of %d at column %d of rows of %d", H, e, col0, ldg);
        return kBadShape;
    }
    const int64_t total = (int64_t)T * H * e;
    if (adtype == kBF16 && e % 8 == 0 && a_head % 8 == 0 && a_tok % 8 == 0 && ldg % 4 == 0 && col0 % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        int64_t vblocks = (total / 8 + 255) / 256;
        if (vblocks > 148 * 16) vblocks = 148 * 16;
        launch_dependent(sigmoid_gate_bf16x8_kernel, dim3((int)vblocks), dim3(256), 0, stream,
                         (const __nv_bfloat16*)a, a_head, a_tok, g, ldg, col0, (__nv_bfloat16*)out, T, H, e / 8);
        return finish_launch("sigmoid_gate");
    }
    const int blocks = (int)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
    MI_DISPATCH_1(adtype, AT,
        launch_dependent(sigmoid_gate_kernel<AT>, dim3(blocks), dim3(256), 0, stream, (const AT*)a, a_head, a_tok, g,
                         ldg, col0, (AT*)out, T, H, e));
    return finish_launch("sigmoid_gate");
}

}  // extern "C"
