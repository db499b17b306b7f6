// Linear attention with a decaying matrix state per head, and the gated norm that follows it.
//
//   tuff_linear_attention   per (request, head): S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
//                           S is [dk, dv] in fp32 in the request's state slot; a_t is either one factor
//                           per head (a constant of the layer) or a factor per key channel and token,
//                           a = sigmoid(z)^(1/tau) with z = gate + bias taken per token
//   tuff_gated_group_norm   y = rmsnorm_group(o) * weight * act(gate) * out_scale, groups of any width
//
// Everything that enters the recurrence is fp32: the decay and its logarithm, the outer product, the
// state and the read-out.  The tensor cores have no fp32 kind (tf32 keeps ten mantissa bits), so the
// recurrence runs on FFMA.  q, k and v come from the projections in the activation dtype; an
// activation (silu) and a scale of q are applied when a token's vectors are staged.
//
// One CTA owns (batch row, head, 32 value columns) and walks the row's tokens in order; a thread owns
// one value column and every fourth group of four key channels, so a token costs it dk/4 fused
// multiply-adds on state in registers and two shuffles.  Tokens are staged through shared memory 16 (8 for the widest heads) at
// a time (activation, decay and scale computed once per element there).  The order of all sums depends on
// the sizes only: a request's state and outputs are the same bits however its tokens were cut into steps.
#include "common.cuh"
#include "index.cuh"

namespace {
constexpr int LA_THREADS = 128;         // 4 warps: 32 value columns x 4 key-channel groups
constexpr int LA_COLS = 32;
constexpr int LA_KG = 4;

enum { LA_DECAY_HEAD = 0, LA_DECAY_CHANNEL = 1 };

struct LinAttnParams {
    const void* q; const void* k; const void* v;          // activation dtype, head h at column h*dk (h*dv for v)
    long long q_stride, k_stride, v_stride;               // elements between tokens
    const float* head_decay;                              // [H] (LA_DECAY_HEAD)
    const float* gate; long long gate_stride;             // fp32 [T, H*dk] (LA_DECAY_CHANNEL): z before the bias
    const float* gate_bias;                               // [H*dk] or null
    float inv_tau;
    float q_scale;
    int act;                                              // 1: silu on q, k and v
    float* state;                                         // [slots, H, dk, dv]
    const int* slot_of_row; const int* cu_q;
    float* out; long long out_stride;                     // fp32 [T, H*dv]
    int H, dk, dv, mode;
    Bounds bounds;
};

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// log(sigmoid(z)) = -softplus(-z), computed without overflow for any z
__device__ __forceinline__ float log_sigmoid(float z) {
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// NC: groups of four key channels a thread owns (dk <= 16 * NC)
template <typename T, int NC, int MODE>
__global__ void __launch_bounds__(LA_THREADS)
linear_attention_kernel(LinAttnParams p) {
    constexpr int DKP = 16 * NC;                         // padded key channels
    constexpr int LA_STAGE = NC >= 16 ? 8 : 16;          // tokens staged at a time (48 KB of static shared memory at most)
    __shared__ __align__(16) float sq[LA_STAGE][DKP];
    __shared__ __align__(16) float sk[LA_STAGE][DKP];
    __shared__ __align__(16) float sa[MODE == LA_DECAY_CHANNEL ? LA_STAGE : 1][DKP];
    __shared__ float sv[LA_STAGE][LA_COLS];
    const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * LA_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kg = lane & 3;                              // key-channel group: channels 4 * (kg + 4 * i) .. + 3
    const int j = warp * 8 + (lane >> 2);                 // value column within the tile
    const int col = col0 + j;
    const bool col_ok = col < p.dv;
    pdl_wait();
    pdl_launch_dependents();
    const int t0 = ld_act(p.cu_q + r), t1 = ld_act(p.cu_q + r + 1);
    const long long slot = ld_act(p.slot_of_row + r);
    if (!check_slot(p.bounds, slot)) return;
    float* S = p.state + slot_elem(slot, (size_t)p.H * p.dk * p.dv) + (size_t)h * p.dk * p.dv;
    const T* q = reinterpret_cast<const T*>(p.q) + (size_t)h * p.dk;
    const T* k = reinterpret_cast<const T*>(p.k) + (size_t)h * p.dk;
    const T* v = reinterpret_cast<const T*>(p.v) + (size_t)h * p.dv;

    float st[NC][4];
#pragma unroll
    for (int i = 0; i < NC; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = 4 * (kg + LA_KG * i) + e;
            st[i][e] = (col_ok && c < p.dk) ? S[(size_t)c * p.dv + col] : 0.f;
        }
    const float hd = MODE == LA_DECAY_HEAD ? p.head_decay[h] : 1.f;

    for (int base = t0; base < t1; base += LA_STAGE) {
        const int n = min(LA_STAGE, t1 - base);
        __syncthreads();                                  // the stage before this one has been read
        for (int idx = threadIdx.x; idx < n * DKP; idx += LA_THREADS) {
            const int tt = idx / DKP, c = idx - tt * DKP;
            const size_t t = (size_t)(base + tt);
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (c < p.dk) {
                qv = ld_act(q + t * p.q_stride + c);
                kv = ld_act(k + t * p.k_stride + c);
                if (p.act) { qv = silu_f(qv); kv = silu_f(kv); }
                qv *= p.q_scale;
                if (MODE == LA_DECAY_CHANNEL) {
                    float z = ld_act(p.gate + t * p.gate_stride + (size_t)h * p.dk + c);
                    if (p.gate_bias) z += p.gate_bias[(size_t)h * p.dk + c];
                    av = expf(log_sigmoid(z) * p.inv_tau);
                }
            }
            sq[tt][c] = qv; sk[tt][c] = kv;
            if (MODE == LA_DECAY_CHANNEL) sa[tt][c] = av;
        }
        for (int idx = threadIdx.x; idx < n * LA_COLS; idx += LA_THREADS) {
            const int tt = idx / LA_COLS, c = idx - tt * LA_COLS;
            float vv = 0.f;
            if (col0 + c < p.dv) {
                vv = ld_act(v + (size_t)(base + tt) * p.v_stride + col0 + c);
                if (p.act) vv = silu_f(vv);
            }
            sv[tt][c] = vv;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vv = sv[tt][j];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = 4 * (kg + LA_KG * i);
                const float4 kk = *reinterpret_cast<const float4*>(&sk[tt][c]);
                const float4 qq = *reinterpret_cast<const float4*>(&sq[tt][c]);
                float4 aa = make_float4(hd, hd, hd, hd);
                if (MODE == LA_DECAY_CHANNEL) aa = *reinterpret_cast<const float4*>(&sa[tt][c]);
                st[i][0] = fmaf(aa.x, st[i][0], kk.x * vv);
                st[i][1] = fmaf(aa.y, st[i][1], kk.y * vv);
                st[i][2] = fmaf(aa.z, st[i][2], kk.z * vv);
                st[i][3] = fmaf(aa.w, st[i][3], kk.w * vv);
                acc[0] = fmaf(st[i][0], qq.x, acc[0]);
                acc[1] = fmaf(st[i][1], qq.y, acc[1]);
                acc[2] = fmaf(st[i][2], qq.z, acc[2]);
                acc[3] = fmaf(st[i][3], qq.w, acc[3]);
            }
            float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (kg == 0 && col_ok) p.out[(size_t)(base + tt) * p.out_stride + (size_t)h * p.dv + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < NC; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c = 4 * (kg + LA_KG * i) + e;
                if (c < p.dk) S[(size_t)c * p.dv + col] = st[i][e];
            }
    }
}

// ---- gated group norm -------------------------------------------------------------------------
enum { GATE_NONE = 0, GATE_SIGMOID = 1, GATE_SILU = 2 };

__device__ __forceinline__ float gate_value(float g, int act) {
    if (act == GATE_SIGMOID) return 1.f / (1.f + expf(-g));
    if (act == GATE_SILU) return silu_f(g);
    return 1.f;
}

// One block per (token, group): for wide groups (a norm over all heads at once).
template <typename T>
__global__ void gated_norm_block_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                                        const float* __restrict__ w, int w_len, float eps, int act, float out_scale,
                                        T* __restrict__ out, int width, int group) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, g = blockIdx.y;
    pdl_wait();
    const float* orow = o + (size_t)t * width + (size_t)g * group;
    float ss = 0.f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float x = ld_act(orow + i);
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, scratch);
    pdl_launch_dependents();
    const float scale = rsqrtf(ss / (float)group + eps) * out_scale;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const int e = g * group + i;
        float y = ld_act(orow + i) * scale * w[e % w_len];
        if (act != GATE_NONE) y *= gate_value(ld_act(gate + (size_t)t * gate_stride + e), act);
        out[(size_t)t * width + e] = from_f32<T>(y);
    }
}

// One warp per (token, group): for narrow groups (a norm per head).
template <typename T>
__global__ void __launch_bounds__(128)
gated_norm_warp_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                       const float* __restrict__ w, int w_len, float eps, int act, float out_scale,
                       T* __restrict__ out, int width, int group, long long n_items) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_wait();
    pdl_launch_dependents();
    if (item >= n_items) return;
    const int n_groups = width / group;
    const long long t = item / n_groups;
    const int g = (int)(item - t * n_groups);
    const float* orow = o + (size_t)t * width + (size_t)g * group;
    float ss = 0.f;
    for (int i = lane; i < group; i += 32) {
        const float x = ld_act(orow + i);
        ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)group + eps) * out_scale;
    for (int i = lane; i < group; i += 32) {
        const int e = g * group + i;
        float y = ld_act(orow + i) * scale * w[e % w_len];
        if (act != GATE_NONE) y *= gate_value(ld_act(gate + (size_t)t * gate_stride + e), act);
        out[(size_t)t * width + e] = from_f32<T>(y);
    }
}
}  // namespace

// q, k [n_tokens, >= H*dk], v [n_tokens, >= H*dv] in `dtype` with their row strides; out fp32.
// mode 0: head_decay[H]; mode 1: gate fp32 [n_tokens, H*dk] (+ gate_bias), a = sigmoid(z)^(inv_tau).
extern "C" int tuff_linear_attention(const void* q, long long q_stride, const void* k, long long k_stride,
                                     const void* v, long long v_stride, int dtype, int mode, const float* head_decay,
                                     const float* gate, long long gate_stride, const float* gate_bias, float inv_tau,
                                     float q_scale, int act, float* state, long long n_slots, const int* slot_of_row,
                                     const int* cu_q, float* out, long long out_stride, int n_rows, int H, int dk, int dv,
                                     int* status, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H < 1 || H > 65535 || dk < 1 || dk > 256 || dv < 1 || (mode != LA_DECAY_HEAD && mode != LA_DECAY_CHANNEL)) return TUFF_E_SIZE;
    LinAttnParams p;
    p.q = q; p.k = k; p.v = v; p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride;
    p.head_decay = head_decay; p.gate = gate; p.gate_stride = gate_stride; p.gate_bias = gate_bias; p.inv_tau = inv_tau;
    p.q_scale = q_scale; p.act = act; p.state = state; p.slot_of_row = slot_of_row; p.cu_q = cu_q;
    p.out = out; p.out_stride = out_stride; p.H = H; p.dk = dk; p.dv = dv; p.mode = mode;
    p.bounds = Bounds{(long long)n_rows, n_slots, status};
    const dim3 grid(n_rows, H, ceil_div(dv, LA_COLS));
#define LA_GO(T, NC, MODE) return launch_pdl(linear_attention_kernel<T, NC, MODE>, grid, dim3(LA_THREADS), 0, stream, p)
#define LA_PICK(T, MODE) do { if (dk <= 32) LA_GO(T, 2, MODE); else if (dk <= 64) LA_GO(T, 4, MODE); \
        else if (dk <= 128) LA_GO(T, 8, MODE); else LA_GO(T, 16, MODE); } while (0)
    if (dtype == TUFF_F32) { if (mode == LA_DECAY_HEAD) LA_PICK(float, LA_DECAY_HEAD); else LA_PICK(float, LA_DECAY_CHANNEL); }
    if (dtype == TUFF_BF16) { if (mode == LA_DECAY_HEAD) LA_PICK(bf16, LA_DECAY_HEAD); else LA_PICK(bf16, LA_DECAY_CHANNEL); }
#undef LA_PICK
#undef LA_GO
    return TUFF_E_DTYPE;
}

// o fp32 [n_tokens, width]; groups of `group` columns are normed; weight index = column % w_len;
// gate [n_tokens, >= width] in `dtype` (ignored for act 0); out [n_tokens, width] in `dtype`.
extern "C" int tuff_gated_group_norm(const float* o, const void* gate, long long gate_stride, int dtype, const float* w,
                                     int w_len, float eps, int act, float out_scale, void* out, int n_tokens, int width,
                                     int group, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (group < 1 || width % group || w_len < 1 || width / group > 65535) return TUFF_E_SIZE;
    const int n_groups = width / group;
    if (group <= 256) {
        const long long items = (long long)n_tokens * n_groups;
        const dim3 grid((unsigned)((items + 3) / 4));
#define GN_GO(T) return launch_pdl(gated_norm_warp_kernel<T>, grid, dim3(128), 0, stream, o, (const T*)gate, gate_stride, w, w_len, \
        eps, act, out_scale, (T*)out, width, group, items)
        if (dtype == TUFF_F32) GN_GO(float);
        if (dtype == TUFF_BF16) GN_GO(bf16);
#undef GN_GO
        return TUFF_E_DTYPE;
    }
    const dim3 grid(n_tokens, n_groups);
#define GN_GO(T) return launch_pdl(gated_norm_block_kernel<T>, grid, dim3(256), 0, stream, o, (const T*)gate, gate_stride, w, w_len, \
        eps, act, out_scale, (T*)out, width, group)
    if (dtype == TUFF_F32) GN_GO(float);
    if (dtype == TUFF_BF16) GN_GO(bf16);
#undef GN_GO
    return TUFF_E_DTYPE;
}
