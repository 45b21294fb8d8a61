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
// Two kernels. The gates' kernel walks the scalar part once a head: a warp a (request, head) takes 32
// rows at a time, computes their gates side by side, finds the running maximum by a warp scan (the step
// x -> max(x + gf, gi) composes: (a2, b2) after (a1, b1) is (a1 + a2, max(b1 + a2, b2))) and leaves, for
// every row, e^(gf + m - m'), e^(gi - m') and e^(-m'). The memory's kernel then has no exponential left:
// one block = one request of the step x one head x a slice of MV value components, a warp a component,
// lane l the memory's rows j = l, l + 32, ... and the normaliser's same rows in registers (every slice
// keeps a copy of n of its own, so slices never read what another writes). The rows of a request are
// walked in order; their inputs (k, q, the slice's v, the three factors) come into shared memory a
// chunk of rows at a time, every value fetched (and, for split-K partial sums, added up) once a block;
// from a float32 tensor the next chunk arrives by asynchronous copies (16 bytes at a time where the
// product's columns allow) while this one is walked. A slice's part of the memory lies in the state
// table in the order of the threads that hold it, so it is read and written in whole lines; the
// running maximum lies once a head behind the slices.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int MV = 4;           // value components a block
constexpr int MJ = 32;          // threads that share a component: a warp
constexpr int MLSTM_THREADS = MV * MJ;

__device__ __forceinline__ float log_sigmoid(float x) {
    return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x));
}

struct MlstmParams {
    float* out;                 // [rows, heads, e] float32: the read-out, not yet normed
    float* factors;             // [rows, heads, 3] float32: e^(gf + m - m'), e^(gi - m'), e^(-m') of every row
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

// Floats of one slice of one head's state: the memory's rows in the threads' order
// [ceil(d / MJ)][MV * MJ], then the slice's copy of n [d]. A head: its slices, then m.
__host__ __device__ inline long long mlstm_slice_floats(int d) {
    return (long long)((d + MJ - 1) / MJ) * MLSTM_THREADS + d;
}
__host__ __device__ inline long long mlstm_state_floats(int d, int e) {
    return (long long)((e + MV - 1) / MV) * mlstm_slice_floats(d) + 1;
}

__device__ __forceinline__ void mlstm_copy4(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d32), "l"(src) : "memory");
}
__device__ __forceinline__ void mlstm_copy16(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src) : "memory");
}

// One warp a (request, head).
template <typename TS>
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(const Src<TS> src, const MlstmParams p) {
    const int entry = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    if (r1 <= r0) return;
    const int slot = p.slots[entry];
    if (slot <= 0 || slot >= p.n_slots) return;
    float* m_at = p.state + ((size_t)slot * p.heads + head + 1) * mlstm_state_floats(p.d, p.e) - 1;
    float m = *m_at;
    const float bi = p.bias_i[head], bf = p.bias_f[head];
    for (int base = r0; base < r1; base += 32) {
        const int r = base + lane;
        const bool live = r < r1;
        float gi = 0.f, gf = 0.f;
        if (live) {
            const size_t at = (size_t)r * p.row_width;
            gi = p.cap * tanhf((src.at(at + p.i_off + head) + bi) / p.cap);
            gf = log_sigmoid(p.cap * tanhf((src.at(at + p.f_off + head) + bf) / p.cap));
        }
        // the step of row r is x -> max(x + a, b); rows beyond the end are the identity (0, -inf)
        float a = live ? gf : 0.f, b = live ? gi : -INFINITY;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float a1 = __shfl_up_sync(0xffffffffu, a, o), b1 = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) {                                 // (a, b) after (a1, b1)
                b = fmaxf(b1 + a, b);
                a = a1 + a;
            }
        }
        const float m_here = fmaxf(m + a, b);                // the maximum after row r
        float m_before = __shfl_up_sync(0xffffffffu, m_here, 1);
        if (lane == 0) m_before = m;
        if (live) {
            float* f = p.factors + ((size_t)r * p.heads + head) * 3;
            f[0] = expf(gf + m_before - m_here);
            f[1] = expf(gi - m_here);
            f[2] = expf(-m_here);
        }
        m = __shfl_sync(0xffffffffu, m_here, min(31, r1 - 1 - base));
    }
    if (lane == 0) *m_at = m;
}

// R: memory rows a thread holds (d <= R * MJ); CH: rows of the step staged at a time.
template <typename TS, int R, int CH>
__global__ void __launch_bounds__(MLSTM_THREADS)
mlstm_scan_kernel(const Src<TS> src, const MlstmParams p) {
    extern __shared__ __align__(16) float staged[];          // [2][CH][rowf]
    const int entry = blockIdx.x, head = blockIdx.y, slice = blockIdx.z;
    const int tid = threadIdx.x;
    const int cl = tid / MJ, c = slice * MV + cl;
    const int jg = tid % MJ;
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
    float* st = p.state + ((size_t)slot * p.heads + head) * mlstm_state_floats(d, e) + (size_t)slice * mlstm_slice_floats(d);
    float* st_n = st + (size_t)((d + MJ - 1) / MJ) * MLSTM_THREADS;
    float S[R], n[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int j = jg + i * MJ;
        S[i] = j < d ? st[(size_t)i * MLSTM_THREADS + tid] : 0.f;
        n[i] = j < d ? st_n[j] : 0.f;
    }

    constexpr int DP = R * MJ;                               // k and q padded to the threads' rows, zeros beyond d
    constexpr int tail = 2 * DP;                             // v [MV] | the three factors | padding
    constexpr int rowf = 2 * DP + 8;                         // k [DP] | q [DP] | tail
    bool async = false;
    if constexpr (sizeof(TS) == 4) async = src.splits == 1;
    // k and q as 16-byte pieces where every piece starts on a 16-byte boundary on both sides
    const bool wide = async && d % 4 == 0 && p.row_width % 4 == 0 && (p.k_off + head * d) % 4 == 0 && (p.q_off + head * d) % 4 == 0 &&
                      ((uintptr_t)src.p & 15) == 0;
    auto stage = [&](int chunk, int buf) {
        const int rbase = r0 + chunk * CH;
        const int nr = min(CH, r1 - rbase);
        float* base = staged + (size_t)buf * CH * rowf;
        // a warp a row in turn; its lanes walk the row's k, then its q
        for (int t = tid / 32; t < nr; t += MLSTM_THREADS / 32) {
            float* row = base + (size_t)t * rowf;
            const size_t at = (size_t)(rbase + t) * p.row_width + (size_t)head * d;
            const float* g = reinterpret_cast<const float*>(src.p);
            if (wide) {
                for (int x = (tid & 31) * 4; x < d; x += 128) {
                    mlstm_copy16(row + x, g + at + p.k_off + x);
                    mlstm_copy16(row + DP + x, g + at + p.q_off + x);
                }
            } else {
                for (int x = tid & 31; x < d; x += 32) {
                    if (async) {
                        mlstm_copy4(row + x, g + at + p.k_off + x);
                        mlstm_copy4(row + DP + x, g + at + p.q_off + x);
                    } else {
                        row[x] = src.at(at + p.k_off + x);
                        row[DP + x] = src.at(at + p.q_off + x);
                    }
                }
            }
        }
        for (int idx = tid; idx < nr * (MV + 3); idx += MLSTM_THREADS) {
            const int t = idx / (MV + 3), x = idx - t * (MV + 3);
            float* dst = base + (size_t)t * rowf + tail + x;
            if (x < MV) {
                const int cc = slice * MV + x;
                const size_t at = (size_t)(rbase + t) * p.row_width + p.v_off + (size_t)head * e + cc;
                if (cc >= e) *dst = 0.f;
                else if (async) mlstm_copy4(dst, reinterpret_cast<const float*>(src.p) + at);
                else *dst = src.at(at);
            } else {
                const float* f = p.factors + ((size_t)(rbase + t) * p.heads + head) * 3 + (x - MV);
                if (async) mlstm_copy4(dst, f);
                else *dst = *f;
            }
        }
        if (async) asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (d < DP) {                                            // the padding of k and q, once: no copy ever writes it
        for (int idx = tid; idx < 2 * CH * 2 * (DP - d); idx += MLSTM_THREADS) {
            const int t = idx / (2 * (DP - d)), x = idx - t * 2 * (DP - d);
            staged[(size_t)t * rowf + (x < DP - d ? d + x : DP + d + (x - (DP - d)))] = 0.f;
        }
    }
    const int chunks = (r1 - r0 + CH - 1) / CH;
    stage(0, 0);
    for (int ch = 0; ch < chunks; ++ch) {
        if (async) {
            if (ch + 1 < chunks) {
                stage(ch + 1, (ch + 1) & 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        }
        __syncthreads();
        const int rbase = r0 + ch * CH;
        const int nr = min(CH, r1 - rbase);
        const float* rows = staged + (size_t)(ch & 1) * CH * rowf;
        for (int t = 0; t < nr; ++t) {
            const float* in = rows + (size_t)t * rowf;
            const float fa = in[tail + MV], fb = in[tail + MV + 1], em = in[tail + MV + 2];
            const float bv = fb * in[tail + cl];
            float acc[2] = {0.f, 0.f}, nq[2] = {0.f, 0.f};     // two chains each, rows in turn
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const float kk = in[jg + i * MJ];
                const float q = in[DP + jg + i * MJ] * p.q_scale;
                S[i] = fmaf(fa, S[i], kk * bv);
                n[i] = fmaf(fa, n[i], fb * kk);
                acc[i & 1] = fmaf(S[i], q, acc[i & 1]);
                nq[i & 1] = fmaf(n[i], q, nq[i & 1]);
            }
            float a = acc[0] + acc[1], b = nq[0] + nq[1];
#pragma unroll
            for (int o = MJ / 2; o > 0; o >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, o);
                b += __shfl_xor_sync(0xffffffffu, b, o);
            }
            if (live && jg == 0) p.out[((size_t)(rbase + t) * p.heads + head) * e + c] = a * __frcp_rn(fmaxf(fabsf(b), em) + p.floor_);
        }
        __syncthreads();                                     // the chunk's buffer may be written again
        if (!async && ch + 1 < chunks) stage(ch + 1, (ch + 1) & 1);
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int j = jg + i * MJ;
        if (j < d) {
            st[(size_t)i * MLSTM_THREADS + tid] = live ? S[i] : 0.f;
            if (cl == 0) st_n[j] = n[i];                     // the slice's first component writes its copy of n
        }
    }
}

}  // namespace kb

using namespace kb;

extern "C" long long kb_mlstm_state_floats(int d, int e) { return mlstm_state_floats(d, e); }

extern "C" int kb_mlstm_scan(float* out, float* factors, const void* src, int in_dt, int splits, long long split_stride, int row_width,
                             int q_off, int k_off, int v_off, int i_off, int f_off, const float* bias_i, const float* bias_f,
                             float* state, int n_slots, const int* entry_start, const int* entry_end, const int* slots,
                             int entries, int rows, int heads, int d, int e, float cap, float q_scale, float floor_,
                             void* stream) {
    KB_REQUIRE(entries >= 0 && rows >= 0 && heads > 0 && d > 0 && e > 0, "mlstm: entries %d, rows %d, heads %d of %d / %d", entries, rows, heads, d, e);
    KB_REQUIRE(d <= 8 * MJ, "mlstm: a key size of %d is more than the kernel's %d", d, 8 * MJ);
    KB_REQUIRE(cap > 0.f, "mlstm: gate cap %g must be positive", cap);
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + heads * d <= row_width && k_off >= 0 && k_off + heads * d <= row_width &&
                   v_off >= 0 && v_off + heads * e <= row_width && i_off >= 0 && i_off + heads <= row_width && f_off >= 0 &&
                   f_off + heads <= row_width,
               "mlstm: columns q %d, k %d, v %d, i %d, f %d do not fit a row of %d", q_off, k_off, v_off, i_off, f_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "mlstm: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(n_slots >= 1 && state && factors && bias_i && bias_f && entry_start && entry_end && slots, "mlstm: state, scratch, biases or ranges are missing");
    if (entries == 0 || rows == 0) return 0;
    const int slices = (e + MV - 1) / MV;
    KB_REQUIRE(heads <= 65535 && slices <= 65535, "mlstm: too many heads or value components for one launch");
    MlstmParams p;
    p.out = out; p.factors = factors; p.row_width = row_width; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.i_off = i_off; p.f_off = f_off;
    p.bias_i = bias_i; p.bias_f = bias_f; p.state = state; p.entry_start = entry_start; p.entry_end = entry_end; p.slots = slots;
    p.n_slots = n_slots; p.heads = heads; p.d = d; p.e = e; p.slices = slices; p.cap = cap; p.q_scale = q_scale; p.floor_ = floor_;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(entries, heads, slices);
    const int need = (d + MJ - 1) / MJ;
#define KB_MLSTM(TS, R, CH)                                                                                                     \
    do {                                                                                                                        \
        mlstm_gates_kernel<TS><<<dim3(entries, heads), 32, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p);     \
        if (int err = check_launch("mlstm gates")) return err;                                                                  \
        mlstm_scan_kernel<TS, R, CH><<<grid, MLSTM_THREADS, (size_t)2 * CH * (2 * R * MJ + 8) * sizeof(float), s>>>(             \
            Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p);                                                          \
    } while (0)
#define KB_MLSTM_R(TS)                            \
    do {                                          \
        if (need <= 1) KB_MLSTM(TS, 1, 16);       \
        else if (need <= 2) KB_MLSTM(TS, 2, 16);  \
        else if (need <= 4) KB_MLSTM(TS, 4, 16);  \
        else KB_MLSTM(TS, 8, 8);                  \
    } while (0)
    if (in_dt == KB_DT_F32) KB_MLSTM_R(float);
    else if (in_dt == KB_DT_BF16) KB_MLSTM_R(bf16);
    else return fail("mlstm: dtype code %d is not known", in_dt);
#undef KB_MLSTM_R
#undef KB_MLSTM
    return check_launch("mlstm scan");
}
