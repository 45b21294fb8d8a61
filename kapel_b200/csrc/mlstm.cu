// The matrix memory with exponential gates (mLSTM), token by token, over the rows of a step.
//
// For each head, with log input gate gi = cap * tanh(zi / cap) and log forget gate
// gf = logsigmoid(cap * tanh(zf / cap)) (z = projection + bias), and a running maximum m:
//     m' = max(gf + m, gi);  S' = e^(gf + m - m') S + e^(gi - m') k v^T;  n' likewise with k alone;
//     o  = S'^T q / (max(|n' . q|, e^(-m')) + floor),  q scaled by `q_scale`.
// S, n and m live in a slot of a float32 state table, one slot a request, and are carried from the
// last row of a request in this step to its first row in the next. Everything here is 32-bit;
// only the projections may come in bfloat16.
//
// One block = one request of the step x one head x a slice of MV value components. A thread holds
// the memory's rows j = jg, jg + MJ, ... of one value component c, and the normaliser's same rows
// (every slice keeps a copy of n and m of its own, so slices never read what another writes).
// The MJ threads of a component are neighbouring lanes and add up by shuffles. The rows of a
// request are walked in order; the next row's inputs are loaded while this row's are used.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int MV = 16;          // value components a block
constexpr int MJ = 8;           // threads that share a component
constexpr int MLSTM_THREADS = MV * MJ;

__device__ __forceinline__ float log_sigmoid(float x) {
    return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
}

struct MlstmParams {
    float* out;                 // [rows, heads, e] float32: the read-out, not yet normed
    int row_width;              // columns of the stacked product
    int q_off, k_off, v_off, i_off, f_off;
    const float* bias_i;        // [heads]
    const float* bias_f;
    float* state;               // [slots, heads, state_floats]
    const int* entry_start;     // [entries]
    const int* entry_end;
    const int* slots;           // [entries]; slot 0 belongs to rows that are no token's
    int n_slots, heads, d, e, slices;
    float cap, q_scale, floor_;
};

// Floats of one head's state: S [d][e], then a copy of n [d] and of m for every slice.
__host__ __device__ inline long long mlstm_state_floats(int d, int e) {
    const int slices = (e + MV - 1) / MV;
    return (long long)d * e + (long long)slices * (d + 1);
}

template <typename TS, int R>
__global__ void __launch_bounds__(MLSTM_THREADS)
mlstm_scan_kernel(const Src<TS> src, const MlstmParams p) {
    const int entry = blockIdx.x, head = blockIdx.y, slice = blockIdx.z;
    const int c = slice * MV + (threadIdx.x / MJ);
    const int jg = threadIdx.x % MJ;
    const bool live = c < p.e;
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    if (r1 <= r0) return;
    const int slot = p.slots[entry];
    const int d = p.d, e = p.e;
    if (slot <= 0 || slot >= p.n_slots) {                    // rows of no request: zeros, no state
        if (live && jg == 0)
            for (int r = r0; r < r1; ++r) p.out[((size_t)r * p.heads + head) * e + c] = 0.f;
        return;
    }
    float* st = p.state + ((size_t)slot * p.heads + head) * mlstm_state_floats(d, e);
    float* st_n = st + (size_t)d * e + (size_t)slice * (d + 1);
    float S[R], n[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int j = jg + i * MJ;
        S[i] = (live && j < d) ? st[(size_t)j * e + c] : 0.f;
        n[i] = j < d ? st_n[j] : 0.f;
    }
    float m = st_n[d];
    const float bi = p.bias_i[head], bf = p.bias_f[head];

    // Two sets of inputs, taken in turn (named apart, so that both stay in registers).
    float k0[R], q0[R], k1[R], q1[R], v0, v1, zi0, zi1, zf0, zf1;
    auto fetch = [&](int r, float (&kk)[R], float (&qq)[R], float& vv, float& zi, float& zf) {
        const size_t base = (size_t)r * p.row_width;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int j = jg + i * MJ;
            kk[i] = j < d ? src.at(base + p.k_off + (size_t)head * d + j) : 0.f;
            qq[i] = j < d ? src.at(base + p.q_off + (size_t)head * d + j) : 0.f;
        }
        vv = live ? src.at(base + p.v_off + (size_t)head * e + c) : 0.f;
        zi = src.at(base + p.i_off + head);
        zf = src.at(base + p.f_off + head);
    };
    auto step = [&](int r, const float (&kk)[R], const float (&qq)[R], float vv, float zi, float zf) {
        const float gi = p.cap * tanhf((zi + bi) / p.cap);
        const float gf = log_sigmoid(p.cap * tanhf((zf + bf) / p.cap));
        const float m_new = fmaxf(gf + m, gi);
        const float fa = expf(gf + m - m_new);
        const float fb = expf(gi - m_new);
        m = m_new;
        const float bv = fb * vv;
        float acc = 0.f, nq = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const float q = qq[i] * p.q_scale;
            S[i] = fmaf(fa, S[i], kk[i] * bv);
            n[i] = fmaf(fa, n[i], fb * kk[i]);
            acc = fmaf(S[i], q, acc);
            nq = fmaf(n[i], q, nq);
        }
#pragma unroll
        for (int o = MJ / 2; o > 0; o >>= 1) {
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
            nq += __shfl_xor_sync(0xffffffffu, nq, o);
        }
        if (live && jg == 0) {
            const float denom = fmaxf(fabsf(nq), expf(-m)) + p.floor_;
            p.out[((size_t)r * p.heads + head) * e + c] = acc / denom;
        }
    };
    fetch(r0, k0, q0, v0, zi0, zf0);
    for (int r = r0; r < r1; r += 2) {
        if (r + 1 < r1) fetch(r + 1, k1, q1, v1, zi1, zf1);
        step(r, k0, q0, v0, zi0, zf0);
        if (r + 1 >= r1) break;
        if (r + 2 < r1) fetch(r + 2, k0, q0, v0, zi0, zf0);
        step(r + 1, k1, q1, v1, zi1, zf1);
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int j = jg + i * MJ;
        if (j < d) {
            if (live) st[(size_t)j * e + c] = S[i];
            if (threadIdx.x / MJ == 0) st_n[j] = n[i];       // the slice's first component writes its copy of n
        }
    }
    if (threadIdx.x == 0) st_n[d] = m;
}

}  // namespace kb

using namespace kb;

extern "C" long long kb_mlstm_state_floats(int d, int e) { return mlstm_state_floats(d, e); }

extern "C" int kb_mlstm_scan(float* out, const void* src, int in_dt, int splits, long long split_stride, int row_width,
                             int q_off, int k_off, int v_off, int i_off, int f_off, const float* bias_i, const float* bias_f,
                             float* state, int n_slots, const int* entry_start, const int* entry_end, const int* slots,
                             int entries, int rows, int heads, int d, int e, float cap, float q_scale, float floor_,
                             void* stream) {
    KB_REQUIRE(entries >= 0 && rows >= 0 && heads > 0 && d > 0 && e > 0, "mlstm: entries %d, rows %d, heads %d of %d / %d", entries, rows, heads, d, e);
    KB_REQUIRE(d <= 32 * MJ, "mlstm: a key size of %d is more than the kernel's %d", d, 32 * MJ);
    KB_REQUIRE(cap > 0.f, "mlstm: gate cap %g must be positive", cap);
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + heads * d <= row_width && k_off >= 0 && k_off + heads * d <= row_width &&
                   v_off >= 0 && v_off + heads * e <= row_width && i_off >= 0 && i_off + heads <= row_width && f_off >= 0 &&
                   f_off + heads <= row_width,
               "mlstm: columns q %d, k %d, v %d, i %d, f %d do not fit a row of %d", q_off, k_off, v_off, i_off, f_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "mlstm: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(n_slots >= 1 && state && bias_i && bias_f && entry_start && entry_end && slots, "mlstm: state, biases or ranges are missing");
    if (entries == 0 || rows == 0) return 0;
    const int slices = (e + MV - 1) / MV;
    KB_REQUIRE(heads <= 65535 && slices <= 65535, "mlstm: too many heads or value components for one launch");
    MlstmParams p;
    p.out = out; p.row_width = row_width; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.i_off = i_off; p.f_off = f_off;
    p.bias_i = bias_i; p.bias_f = bias_f; p.state = state; p.entry_start = entry_start; p.entry_end = entry_end; p.slots = slots;
    p.n_slots = n_slots; p.heads = heads; p.d = d; p.e = e; p.slices = slices; p.cap = cap; p.q_scale = q_scale; p.floor_ = floor_;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(entries, heads, slices);
    const int need = (d + MJ - 1) / MJ;
#define KB_MLSTM(TS, R) mlstm_scan_kernel<TS, R><<<grid, MLSTM_THREADS, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p)
#define KB_MLSTM_R(TS)                       \
    do {                                     \
        if (need <= 4) KB_MLSTM(TS, 4);      \
        else if (need <= 8) KB_MLSTM(TS, 8); \
        else if (need <= 16) KB_MLSTM(TS, 16); \
        else KB_MLSTM(TS, 32);               \
    } while (0)
    if (in_dt == KB_DT_F32) KB_MLSTM_R(float);
    else if (in_dt == KB_DT_BF16) KB_MLSTM_R(bf16);
    else return fail("mlstm: dtype code %d is not known", in_dt);
#undef KB_MLSTM_R
#undef KB_MLSTM
    return check_launch("mlstm scan");
}
