// What a mixer does around its products and its core, for mixers whose inputs come as one stacked
// product [rows, row_width] (a tensor or split-K partial sums) with each role at a column offset:
//
//  proj_norm_append  an RMS norm over the whole query projection and over the whole key projection
//                    (all heads' components of a row at once), the queries written out as
//                    [rows, hq, d], keys and values written to the paged cache at each row's line.
//                    The counterpart of rotate-and-append for a mixer without a rotation.
//  head_gate         y[r, h, :] (optionally divided by its root mean square over the head, times a
//                    weight over all heads) times sigmoid(gate[r, h, :]), the gate read from the
//                    stacked product; the output's rows may be wider than the heads (zeros behind them).
//  entry_ranges      first row and one past the last row of every request of a step, from the rows' entries.
//
// Sums, norms and the sigmoid are 32-bit.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

template <typename TS, typename TW, typename TO>
__global__ void proj_norm_append_kernel(const Src<TS> src, int row_width, int q_off, int k_off, int v_off,
                                        const TW* __restrict__ wq, float eps_q, float off_q,
                                        const TW* __restrict__ wk, float eps_k, float off_k,
                                        const int* __restrict__ lines, TO* __restrict__ q_out, TO* __restrict__ k_table,
                                        TO* __restrict__ v_table, int hq, int hkv, int d, int dv, long long table_lines,
                                        int page_size) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t base = (size_t)r * row_width;
    const int nq = hq * d, nk = hkv * d, nv = hkv * dv;
    float inv_q = 1.f, inv_k = 1.f;
    if (wq != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) {
            const float v = src.at(base + q_off + i);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_q = 1.f / sqrtf(ss / (float)nq + eps_q);
    }
    if (wk != nullptr) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float v = src.at(base + k_off + i);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_k = 1.f / sqrtf(ss / (float)nk + eps_k);
    }
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        float v = src.at(base + q_off + i);
        if (wq != nullptr) v = v * inv_q * (off_q + Elem<TW>::load(wq + i));
        Elem<TO>::store(q_out + (size_t)r * nq + i, v);
    }
    if (k_table == nullptr) return;
    const long long line = lines[r];
    if (line < 0 || line >= table_lines) return;          // a row that writes nowhere (padding)
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        float v = src.at(base + k_off + i);
        if (wk != nullptr) v = v * inv_k * (off_k + Elem<TW>::load(wk + i));
        const int h = i / d, c = i - h * d;
        Elem<TO>::store(k_table + kv_row(line, h, hkv, page_size) * d + c, v);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        Elem<TO>::store(v_table + kv_row(line, h, hkv, page_size) * dv + c, src.at(base + v_off + i));
    }
}

// One warp a (row, head).
template <typename TY, typename TS, typename TW, typename TO>
__global__ void head_gate_kernel(TO* __restrict__ out, const TY* __restrict__ y, const Src<TS> gate, int row_width,
                                 int g_off, const TW* __restrict__ w, int unit, float eps, long long pairs, int heads, int e,
                                 int out_stride) {
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int lane = threadIdx.x & 31;
    const long long r = pair / heads;
    const int h = (int)(pair - r * heads);
    const TY* yp = y + (size_t)pair * e;
    float inv = 1.f;
    if (unit) {
        float ss = 0.f;
        for (int c = lane; c < e; c += 32) {
            const float v = Elem<TY>::load(yp + c);
            ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)e + eps);
    }
    for (int c = lane; c < e; c += 32) {
        float v = Elem<TY>::load(yp + c) * inv;
        if (w != nullptr) v *= Elem<TW>::load(w + (size_t)h * e + c);
        const float z = gate.at((size_t)r * row_width + g_off + (size_t)h * e + c);
        v *= 1.f / (1.f + expf(-z));
        Elem<TO>::store(out + (size_t)r * out_stride + (size_t)h * e + c, v);
    }
    // a row wider than its heads (padding for the product that follows) ends in zeros
    if (h == heads - 1)
        for (int c = heads * e + lane; c < out_stride; c += 32) Elem<TO>::store(out + (size_t)r * out_stride + c, 0.f);
}

__global__ void entry_ranges_clear_kernel(int entries, int* __restrict__ start, int* __restrict__ end) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < entries) {                                      // an entry without rows keeps the empty range
        start[i] = 0;
        end[i] = 0;
    }
}
__global__ void entry_ranges_fill_kernel(const int* __restrict__ row_entry, int rows, int entries, int* __restrict__ start,
                                         int* __restrict__ end) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int e = row_entry[r];
    if (e < 0 || e >= entries) return;
    if (r == 0 || row_entry[r - 1] != e) start[e] = r;
    if (r == rows - 1 || row_entry[r + 1] != e) end[e] = r + 1;
}

}  // namespace kb

using namespace kb;

// Rows [start[e], end[e]) are entry e's (the rows of one entry lie together). Two launches.
extern "C" int kb_entry_ranges(int* start, int* end, const int* row_entry, int rows, int entries, void* stream) {
    KB_REQUIRE(rows >= 0 && entries >= 0, "entry_ranges: rows %d, entries %d", rows, entries);
    if (entries == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    entry_ranges_clear_kernel<<<(entries + 255) / 256, 256, 0, s>>>(entries, start, end);
    if (int e = check_launch("entry_ranges")) return e;
    if (rows == 0) return 0;
    entry_ranges_fill_kernel<<<(rows + 255) / 256, 256, 0, s>>>(row_entry, rows, entries, start, end);
    return check_launch("entry_ranges");
}

extern "C" int kb_proj_norm_append(const void* src, int in_dt, int splits, long long split_stride, int row_width, int q_off,
                                   int k_off, int v_off, const void* wq, float eps_q, float off_q, const void* wk,
                                   float eps_k, float off_k, int w_dt, const int* lines, void* q_out, void* k_table,
                                   void* v_table, int out_dt, int rows, int hq, int hkv, int d, int dv, int write_kv,
                                   long long table_lines, int page_size, void* stream) {
    KB_REQUIRE(rows >= 0 && hq > 0 && hkv > 0 && d > 0 && dv > 0, "proj_norm_append: rows %d, heads %d / %d, sizes %d / %d", rows, hq, hkv, d, dv);
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + hq * d <= row_width && k_off >= 0 && k_off + hkv * d <= row_width &&
                   v_off >= 0 && v_off + hkv * dv <= row_width,
               "proj_norm_append: columns q %d, k %d, v %d do not fit a row of %d", q_off, k_off, v_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "proj_norm_append: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(!write_kv || (lines && k_table && v_table && table_lines > 0 && page_size > 0), "proj_norm_append: no cache to write");
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    void* kt = write_kv ? k_table : nullptr;
    const int threads = 256;
#define KB_PNA(TS, TW, TO)                                                                                              \
    proj_norm_append_kernel<TS, TW, TO><<<rows, threads, 0, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, row_width, q_off, \
                                                                 k_off, v_off, (const TW*)wq, eps_q, off_q, (const TW*)wk, eps_k, off_k, \
                                                                 lines, (TO*)q_out, (TO*)kt, (TO*)v_table, hq, hkv, d, dv, table_lines, page_size)
    const int code = in_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_PNA(float, float, float); break;
        case 1: KB_PNA(float, float, bf16); break;
        case 2: KB_PNA(float, bf16, float); break;
        case 3: KB_PNA(float, bf16, bf16); break;
        case 4: KB_PNA(bf16, float, float); break;
        case 5: KB_PNA(bf16, float, bf16); break;
        case 6: KB_PNA(bf16, bf16, float); break;
        case 7: KB_PNA(bf16, bf16, bf16); break;
        default: return fail("proj_norm_append: dtype codes in %d, w %d, out %d are not known", in_dt, w_dt, out_dt);
    }
#undef KB_PNA
    return check_launch("proj_norm_append");
}

extern "C" int kb_head_gate(void* out, int out_dt, const void* y, int y_dt, const void* gate, int g_dt, int splits,
                            long long split_stride, int row_width, int g_off, const void* w, int w_dt, int unit, float eps,
                            long long rows, int heads, int e, int out_stride, void* stream) {
    KB_REQUIRE(rows >= 0 && heads > 0 && e > 0, "head_gate: rows %lld, heads %d of %d", rows, heads, e);
    KB_REQUIRE(out_stride >= heads * e, "head_gate: output rows of %d values for %d heads of %d", out_stride, heads, e);
    KB_REQUIRE(row_width > 0 && g_off >= 0 && g_off + heads * e <= row_width, "head_gate: gate columns %d.. do not fit a row of %d", g_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= rows * row_width), "head_gate: %d slices %lld apart", splits, split_stride);
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long pairs = rows * heads;
    const int warps = 4;
    const long long blocks = (pairs + warps - 1) / warps;
    KB_REQUIRE(blocks <= 0x7fffffffll, "head_gate: too many rows for one launch");
#define KB_HG(TY, TS, TW, TO)                                                                                       \
    head_gate_kernel<TY, TS, TW, TO><<<(unsigned)blocks, warps * 32, 0, s>>>((TO*)out, (const TY*)y,                    \
                                                                             Src<TS>{(const TS*)gate, splits, (size_t)split_stride}, \
                                                                             row_width, g_off, (const TW*)w, unit, eps, pairs, heads, e, out_stride)
    const int code = y_dt * 8 + g_dt * 4 + w_dt * 2 + out_dt;
    switch (code) {
        case 0: KB_HG(float, float, float, float); break;
        case 1: KB_HG(float, float, float, bf16); break;
        case 2: KB_HG(float, float, bf16, float); break;
        case 3: KB_HG(float, float, bf16, bf16); break;
        case 4: KB_HG(float, bf16, float, float); break;
        case 5: KB_HG(float, bf16, float, bf16); break;
        case 6: KB_HG(float, bf16, bf16, float); break;
        case 7: KB_HG(float, bf16, bf16, bf16); break;
        case 8: KB_HG(bf16, float, float, float); break;
        case 9: KB_HG(bf16, float, float, bf16); break;
        case 10: KB_HG(bf16, float, bf16, float); break;
        case 11: KB_HG(bf16, float, bf16, bf16); break;
        case 12: KB_HG(bf16, bf16, float, float); break;
        case 13: KB_HG(bf16, bf16, float, bf16); break;
        case 14: KB_HG(bf16, bf16, bf16, float); break;
        case 15: KB_HG(bf16, bf16, bf16, bf16); break;
        default: return fail("head_gate: dtype codes y %d, gate %d, w %d, out %d are not known", y_dt, g_dt, w_dt, out_dt);
    }
#undef KB_HG
    return check_launch("head_gate");
}
