// CSR + CSR element-wise kernels: sorted union (add) and intersection (multiply) of two CSR
// operands, as flat merge-path over the (row, column) order.
//
// The merged sequence of all stored entries of A and B, ordered by (row, column) with A first
// on ties, is cut into tiles of TILE_STEP entries. A partition kernel finds every cut with
// warp-wide 32-ary searches (rows on the summed row offsets, then the merge-path diagonal
// inside the row). One CTA then owns one tile: it stages the tile's column indices and values
// in shared memory with coalesced loads, turns them into composite (row-in-tile, column) keys
// so that row boundaries need no special casing, splits the tile among its threads with an
// in-shared-memory merge-path search, merges VT entries per thread in registers, compacts
// the survivors with a CTA scan and writes them back coalesced. Row offsets of the result are
// produced by the same pass: a tile owns the offsets of the rows that begin inside it.
//
// Reference behaviour restated (not its code): partition src/backend/partition.cpp:813-993
// (equal columns never split, :964-983), count src/backend/compute.cpp:152-271, fill
// :273-411, value expressions :426-440, empty-result path
// src/backend/stitch_and_generate.cpp:168-220.
#include <algorithm>

#include "block_utils.cuh"
#include "common.cuh"

namespace nb200 {

namespace {

constexpr int NT = 256;

enum SetOp { OP_UNION = 0, OP_INTERSECT = 1 };
enum Pass { PASS_COUNT = 0, PASS_FILL = 1 };

struct CsrIn {
    const int32_t *rp;
    const int32_t *col;
    const float *val;
    int32_t nnz;
};

struct CsrOut {
    int32_t *rp;
    int32_t *col;
    float *val;
};

// Tile cuts: for cut t, the row it falls in and the absolute positions in A and B.
struct Cuts {
    int32_t *row;
    int32_t *a;
    int32_t *b;
};

// ------------------------------------------------------------------------- partition ----

// One warp per cut. Cut t sits at merged position min(t * tile_step, total).
__global__ void __launch_bounds__(NT) k_csr2_partition(CsrIn A, CsrIn B, int32_t rows, int64_t total,
                                                       int32_t tile_step, int32_t num_tiles, Cuts cuts) {
    const int t = (blockIdx.x * NT + threadIdx.x) >> 5;
    if (t > num_tiles) return;
    const int32_t a_base = ld_nc(A.rp), b_base = ld_nc(B.rp);
    int64_t d = (int64_t)t * tile_step;
    int32_t row, pa, pb;
    if (t == 0) {
        row = 0;
        pa = a_base;
        pb = b_base;
    } else if (t == num_tiles || d >= total) {
        row = rows;
        pa = a_base + A.nnz;
        pb = b_base + B.nnz;
    } else {
        // Row holding merged position d: the largest i with work(i) <= d, where work(i) is the
        // number of entries of A and B in rows before i.
        auto work = [&](int64_t i) -> int64_t {
            return (int64_t)(ld_nc(A.rp + i) - a_base) + (int64_t)(ld_nc(B.rp + i) - b_base);
        };
        row = (int32_t)warp_last_true(0, (int64_t)rows - 1, [&](int64_t i) { return work(i) <= d; });
        const int32_t a_lo = ld_nc(A.rp + row), a_hi = ld_nc(A.rp + row + 1);
        const int32_t b_lo = ld_nc(B.rp + row), b_hi = ld_nc(B.rp + row + 1);
        const int64_t dd = d - ((int64_t)(a_lo - a_base) + (int64_t)(b_lo - b_base));
        const int64_t len_a = a_hi - a_lo, len_b = b_hi - b_lo;
        // Merge-path diagonal dd inside the row: x entries of A and dd - x of B come first.
        const int64_t x_lo = dd - len_b > 0 ? dd - len_b : 0;
        const int64_t x_hi = dd < len_a ? dd : len_a;
        const int64_t x = warp_count_true(x_lo, x_hi, [&](int64_t m) {
            return ld_nc(A.col + a_lo + m) <= ld_nc(B.col + b_lo + (dd - 1 - m));
        });
        int64_t y = dd - x;
        // Keep a column present in both operands on one side of the cut.
        if (x > 0 && y < len_b && ld_nc(A.col + a_lo + x - 1) == ld_nc(B.col + b_lo + y)) ++y;
        pa = a_lo + (int32_t)x;
        pb = b_lo + (int32_t)y;
    }
    if (lane_id() == 0) {
        cuts.row[t] = row;
        cuts.a[t] = pa;
        cuts.b[t] = pb;
    }
}

// ------------------------------------------------------------------------ tile kernel ----

template <typename KeyT>
struct KeyTraits;

template <>
struct KeyTraits<uint32_t> {
    static constexpr uint32_t INF = 0xffffffffu;
    __device__ static __forceinline__ uint32_t row_of(uint32_t k, int cbits) { return k >> cbits; }
    __device__ static __forceinline__ uint32_t col_of(uint32_t k, int cbits) { return k & ((1u << cbits) - 1u); }
    __device__ static __forceinline__ uint32_t make(uint32_t row, uint32_t col, int cbits) { return (row << cbits) | col; }
};

template <>
struct KeyTraits<uint64_t> {
    static constexpr uint64_t INF = ~0ull;
    __device__ static __forceinline__ uint32_t row_of(uint64_t k, int) { return (uint32_t)(k >> 32); }
    __device__ static __forceinline__ uint32_t col_of(uint64_t k, int) { return (uint32_t)k; }
    __device__ static __forceinline__ uint64_t make(uint32_t row, uint32_t col, int) { return ((uint64_t)row << 32) | col; }
};

// Writes `value` into out_rp[first .. last] (inclusive), the whole warp cooperating.
__device__ __forceinline__ void warp_fill_rows(int32_t *out_rp, int64_t first, int64_t last, int32_t value) {
    for (int64_t r = first + lane_id(); r <= last; r += 32) out_rp[r] = value;
}

template <typename KeyT, int VT, int OP, int PASS>
__device__ __forceinline__ void csr2_tile_body(const CsrIn &A, const CsrIn &B, const Cuts &cuts, int cbits,
                                               int32_t *tile_count, const CsrOut &Z, unsigned char *smem_raw,
                                               int *scan_tmp) {
    using KT = KeyTraits<KeyT>;
    constexpr int CAP = NT * VT;  // most merged entries a tile can hold
    const int tid = threadIdx.x;
    const int t = blockIdx.x;
    const int32_t i0 = cuts.row[t], i1 = cuts.row[t + 1];
    const int32_t a0 = cuts.a[t], b0 = cuts.b[t];
    const int na = cuts.a[t + 1] - a0, nb = cuts.b[t + 1] - b0;
    const int n = na + nb;

    KeyT *keys = reinterpret_cast<KeyT *>(smem_raw);  // [0, na) from A, [na, n) from B
    float *vals = reinterpret_cast<float *>(smem_raw + sizeof(KeyT) * (CAP + 2));

    // ---- stage columns (and values) in shared memory, coalesced
    for (int i = tid; i < na; i += NT) keys[i] = (KeyT)(uint32_t)ld_nc(A.col + a0 + i);
    for (int i = tid; i < nb; i += NT) keys[na + i] = (KeyT)(uint32_t)ld_nc(B.col + b0 + i);
    if (PASS == PASS_FILL) {
        for (int i = tid; i < na; i += NT) vals[i] = ld_nc(A.val + a0 + i);
        for (int i = tid; i < nb; i += NT) vals[na + i] = ld_nc(B.val + b0 + i);
    }
    __syncthreads();

    // ---- mark the first entry of every row that starts inside the tile with its row number
    // relative to i0 (max wins where empty rows share a start), then spread it forward with a
    // running maximum so that every entry carries its row in the high bits of its key.
    for (int64_t r = (int64_t)i0 + 1 + tid; r <= i1; r += NT) {
        const uint32_t rr = (uint32_t)(r - i0);
        const int64_t sa = (int64_t)ld_nc(A.rp + r) - a0;
        if (sa >= 0 && sa < na) {
            if (sizeof(KeyT) == 4) atomicMax(reinterpret_cast<unsigned *>(keys) + sa, (rr << cbits) | (unsigned)keys[sa] & ((1u << cbits) - 1u));
            else atomicMax(reinterpret_cast<unsigned *>(keys) + 2 * sa + 1, rr);
        }
        const int64_t sb = (int64_t)ld_nc(B.rp + r) - b0;
        if (sb >= 0 && sb < nb) {
            if (sizeof(KeyT) == 4) atomicMax(reinterpret_cast<unsigned *>(keys) + na + sb, (rr << cbits) | (unsigned)keys[na + sb] & ((1u << cbits) - 1u));
            else atomicMax(reinterpret_cast<unsigned *>(keys) + 2 * (na + sb) + 1, rr);
        }
    }
    __syncthreads();
    {
        const int lo = tid * VT, hi = min(lo + VT, n);
        unsigned ma = 0, mb = 0;
        for (int i = lo; i < hi; ++i) {
            const unsigned rr = KT::row_of(keys[i], cbits);
            if (i < na) ma = max(ma, rr); else mb = max(mb, rr);
        }
        unsigned ea, eb;
        block_excl_max2<NT>(ma, mb, reinterpret_cast<unsigned *>(scan_tmp), ea, eb);
        for (int i = lo; i < hi; ++i) {
            const KeyT k = keys[i];
            const unsigned rr = KT::row_of(k, cbits);
            if (i < na) {
                ea = max(ea, rr);
                keys[i] = KT::make(ea, KT::col_of(k, cbits), cbits);
            } else {
                eb = max(eb, rr);
                keys[i] = KT::make(eb, KT::col_of(k, cbits), cbits);
            }
        }
    }
    __syncthreads();

    // ---- split the tile among threads: merge-path diagonal tid * VT, ties take A first
    const KeyT *kx = keys, *ky = keys + na;
    const int diag = min(tid * VT, n);
    int x, y;
    {
        int lo = max(0, diag - nb), hi = min(diag, na);
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (kx[mid] <= ky[diag - 1 - mid]) lo = mid + 1; else hi = mid;
        }
        x = lo;
        y = diag - lo;
    }

    // ---- merge VT entries in registers
    KeyT key[VT];
    float val[VT];
    unsigned emit = 0;
    KeyT prev_any = KT::INF;  // key of the merged entry just before this thread's first
    {
        KeyT hx = x < na ? kx[x] : KT::INF;
        KeyT hy = y < nb ? ky[y] : KT::INF;
        KeyT last_x = x > 0 ? kx[x - 1] : KT::INF;
        const KeyT last_y = y > 0 ? ky[y - 1] : KT::INF;
        if (x > 0 && y > 0) prev_any = max(last_x, last_y);
        else if (x > 0) prev_any = last_x;
        else if (y > 0) prev_any = last_y;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool valid = diag + i < n;
            const bool take_x = hx <= hy;
            if (take_x) {
                const bool both = hx == hy;
                key[i] = hx;
                if (PASS == PASS_FILL && valid) {
                    const float va = vals[x];
                    if (OP == OP_UNION) val[i] = both ? va + vals[na + y] : va;
                    else val[i] = both ? va * vals[na + y] : 0.f;
                }
                if (valid && (OP == OP_UNION || both)) emit |= 1u << i;
                last_x = hx;
                ++x;
                hx = x < na ? kx[x] : KT::INF;
            } else {
                key[i] = hy;
                if (PASS == PASS_FILL && valid) val[i] = vals[na + y];
                if (valid && OP == OP_UNION && hy != last_x) emit |= 1u << i;
                ++y;
                hy = y < nb ? ky[y] : KT::INF;
            }
        }
    }

    // ---- rank the survivors
    int total;
    const int mine = __popc(emit);
    int rank = block_excl_sum<NT>(mine, scan_tmp, total);  // syncs: all reads of keys/vals are done
    if (PASS == PASS_COUNT) {
        if (tid == 0) tile_count[t] = total;
        return;
    }

    const int32_t base = tile_count[t];  // exclusive prefix over tiles, made between the passes

    // ---- row offsets: an entry that opens a new row closes every row before it
    {
        uint32_t prev_row = prev_any == KT::INF ? 0u : KT::row_of(prev_any, cbits);
        int r = rank;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool valid = diag + i < n;
            const uint32_t row = valid ? KT::row_of(key[i], cbits) : prev_row;
            const uint32_t gap = row - prev_row;
            if (gap > 0 && gap <= 32) {
                for (uint32_t g = 1; g <= gap; ++g) Z.rp[(int64_t)i0 + prev_row + g] = base + r;
            }
            unsigned big = __ballot_sync(FULL_MASK, gap > 32);
            while (big) {
                const int src = __ffs(big) - 1;
                big &= big - 1;
                const uint32_t p = __shfl_sync(FULL_MASK, prev_row, src);
                const uint32_t q = __shfl_sync(FULL_MASK, row, src);
                const int v = __shfl_sync(FULL_MASK, r, src);
                warp_fill_rows(Z.rp, (int64_t)i0 + p + 1, (int64_t)i0 + q, base + v);
            }
            prev_row = row;
            r += (emit >> i) & 1u;
        }
        // the thread holding the tile's last entry closes the rows up to the next tile's first
        const bool owns_last = diag < n && diag + VT >= n;
        const uint32_t end_row = (uint32_t)(i1 - i0);
        unsigned tail = __ballot_sync(FULL_MASK, owns_last && end_row > prev_row);
        if (tail) {
            const int src = __ffs(tail) - 1;
            const uint32_t p = __shfl_sync(FULL_MASK, prev_row, src);
            warp_fill_rows(Z.rp, (int64_t)i0 + p + 1, (int64_t)i0 + end_row, base + total);
        }
        if (t == 0 && tid == 0) Z.rp[0] = 0;
    }

    // ---- compact through shared memory (the staging area reuses the key/value arrays; the
    // scan above already separated the last read from the first write) and store coalesced
    int32_t *out_col = reinterpret_cast<int32_t *>(smem_raw);
    float *out_val = reinterpret_cast<float *>(smem_raw) + (CAP + 2);
    {
        int r = rank;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            if ((emit >> i) & 1u) {
                out_col[r] = (int32_t)KT::col_of(key[i], cbits);
                out_val[r] = val[i];
                ++r;
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < total; i += NT) {
        Z.col[(int64_t)base + i] = out_col[i];
        Z.val[(int64_t)base + i] = out_val[i];
    }
}

template <int VT, int OP, int PASS>
__global__ void __launch_bounds__(NT) k_csr2_tile(CsrIn A, CsrIn B, Cuts cuts, int cbits, int32_t *tile_count, CsrOut Z) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int scan_tmp[72];
    const int t = blockIdx.x;
    // 32-bit composite keys hold (row in tile << cbits | column) when that fits; tiles that
    // span too many rows for that (long runs of empty rows) fall back to 64-bit keys.
    const uint64_t nr = (uint64_t)(cuts.row[t + 1] - cuts.row[t]) + 1;
    const bool narrow = cbits < 32 && (nr << cbits) < 0xffffffffull;
    if (narrow) csr2_tile_body<uint32_t, VT, OP, PASS>(A, B, cuts, cbits, tile_count, Z, smem_raw, scan_tmp);
    else csr2_tile_body<uint64_t, VT, OP, PASS>(A, B, cuts, 32, tile_count, Z, smem_raw, scan_tmp);
}

// Exclusive prefix of the per-tile counts, in place, by one CTA; the grand total goes to
// *total_out (64-bit so that the host can detect int32 overflow).
__global__ void __launch_bounds__(1024) k_scan_tiles(int32_t *counts, int32_t n, int64_t *total_out) {
    __shared__ long long warp_sums[33];
    __shared__ long long carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const long long v = i < n ? counts[i] : 0;
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            long long nb = __shfl_up_sync(FULL_MASK, incl, o);
            if (lane_id() >= o) incl += nb;
        }
        if (lane_id() == 31) warp_sums[warp_id()] = incl;
        __syncthreads();
        if (warp_id() == 0) {
            long long w = warp_sums[lane_id()];
            long long wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                long long nb = __shfl_up_sync(FULL_MASK, wi, o);
                if (lane_id() >= o) wi += nb;
            }
            warp_sums[lane_id()] = wi - w;
            if (lane_id() == 31) warp_sums[32] = wi;
        }
        __syncthreads();
        const long long carry = carry_s;
        const long long excl = carry + warp_sums[warp_id()] + incl - v;
        if (i < n) counts[i] = (int32_t)min(excl, (long long)INT32_MAX);
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + warp_sums[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) *total_out = carry_s;
}

// ------------------------------------------------------------------------ host driver ----

constexpr int VT_CSR2 = 11;

template <int VT>
constexpr size_t csr2_smem_bytes() {
    return (sizeof(uint64_t) + sizeof(float)) * (size_t)(NT * VT + 2);
}

int col_bits(int32_t cols) {
    int b = 1;
    while (b < 32 && (int64_t(1) << b) < (int64_t)cols) ++b;
    return b;
}

int check_csr(const nb200_csr *m, bool need_arrays) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0) return NB200_E_BADARG;
    if (need_arrays && (!m->row_ptr || (m->nnz > 0 && (!m->col || !m->val)))) return NB200_E_BADARG;
    return NB200_OK;
}

template <int OP, int PASS>
cudaError_t launch_tile(const CsrIn &A, const CsrIn &B, const Cuts &cuts, int cbits, int32_t *tile_count,
                        const CsrOut &Z, int num_tiles, cudaStream_t stream) {
    constexpr size_t smem = csr2_smem_bytes<VT_CSR2>();
    auto kernel = k_csr2_tile<VT_CSR2, OP, PASS>;
    static bool configured[64] = {};  // per instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    LaunchScope scope(PASS == PASS_COUNT ? (OP == OP_UNION ? "csr_add_count" : "csr_mul_count")
                                         : (OP == OP_UNION ? "csr_add_fill" : "csr_mul_fill"),
                      stream);
    kernel<<<num_tiles, NT, smem, stream>>>(A, B, cuts, cbits, tile_count, Z);
    return cudaGetLastError();
}

// Shared driver of add and multiply. When `alloc` is set the result arrays are allocated
// here (one cudaMallocAsync each); otherwise z's arrays are the caller's, `capacity` entries.
template <int OP>
int csr2_run(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, bool alloc, int64_t capacity, void *stream_v) {
    int st;
    if ((st = check_csr(a, true)) || (st = check_csr(b, true))) return st;
    if (!z || a->rows != b->rows || a->cols != b->cols) return NB200_E_BADARG;
    if (!alloc && (!z->row_ptr || capacity < 0)) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows;
    const int64_t total = (int64_t)a->nnz + b->nnz;
    constexpr int tile_step = NT * VT_CSR2 - 1;
    const int64_t tiles64 = (total + tile_step - 1) / tile_step;
    if (tiles64 > INT32_MAX - 1) return NB200_E_OVERFLOW;
    const int num_tiles = (int)tiles64;

    z->rows = rows;
    z->cols = a->cols;
    z->nnz = 0;
    if (alloc) {
        z->row_ptr = nullptr;
        z->col = nullptr;
        z->val = nullptr;
        NB200_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&z->row_ptr), sizeof(int32_t) * ((size_t)rows + 1), stream));
    }
    auto fail = [&](int code) {
        if (alloc) {
            cudaFreeAsync(z->row_ptr, stream);
            if (z->col) cudaFreeAsync(z->col, stream);
            if (z->val) cudaFreeAsync(z->val, stream);
            z->row_ptr = z->col = nullptr;
            z->val = nullptr;
        }
        return code;
    };
    if (num_tiles == 0) {  // both operands empty: all-zero offsets, nothing else
        cudaError_t e = cudaMemsetAsync(z->row_ptr, 0, sizeof(int32_t) * ((size_t)rows + 1), stream);
        if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMemsetAsync"));
        return NB200_OK;
    }

    Carver sizes;
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int64_t>(1);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws))) return fail(st);
    Carver carve(ws->dev);
    Cuts cuts;
    cuts.row = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.a = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.b = carve.take<int32_t>((size_t)num_tiles + 1);
    int32_t *tile_count = carve.take<int32_t>((size_t)num_tiles + 1);
    int64_t *d_total = carve.take<int64_t>(1);

    const CsrIn A{a->row_ptr, a->col, a->val, a->nnz}, B{b->row_ptr, b->col, b->val, b->nnz};
    const int cbits = col_bits(a->cols);
    cudaError_t e;
    {
        LaunchScope scope("csr2_partition", stream);
        const int warps = num_tiles + 1;
        const int blocks = (warps * 32 + NT - 1) / NT;
        k_csr2_partition<<<blocks, NT, 0, stream>>>(A, B, rows, total, tile_step, num_tiles, cuts);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_partition"));
    e = launch_tile<OP, PASS_COUNT>(A, B, cuts, cbits, tile_count, CsrOut{nullptr, nullptr, nullptr}, num_tiles, stream);
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_tile<count>"));
    {
        LaunchScope scope("scan_tiles", stream);
        k_scan_tiles<<<1, 1024, 0, stream>>>(tile_count, num_tiles, d_total);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_scan_tiles"));
    e = cudaMemcpyAsync(ws->host, d_total, sizeof(int64_t), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(note_cuda_error(e, "read result length"));
    const int64_t nnz = ws->host[0];
    if (nnz > INT32_MAX) return fail(NB200_E_OVERFLOW);
    z->nnz = (int32_t)nnz;

    if (alloc) {
        if (nnz > 0) {
            e = cudaMallocAsync(reinterpret_cast<void **>(&z->col), sizeof(int32_t) * (size_t)nnz, stream);
            if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&z->val), sizeof(float) * (size_t)nnz, stream);
            if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMallocAsync"));
        }
    } else if (nnz > capacity) {
        return NB200_E_CAPACITY;
    }
    e = launch_tile<OP, PASS_FILL>(A, B, cuts, cbits, tile_count, CsrOut{z->row_ptr, z->col, z->val}, num_tiles, stream);
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_tile<fill>"));
    return NB200_OK;
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_csr_add_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int32_t, int32_t, void *stream) {
    return csr2_run<OP_UNION>(a, b, z, true, 0, stream);
}

int nb200_csr_add_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream) {
    return csr2_run<OP_UNION>(a, b, z, false, capacity, stream);
}

int nb200_csr_mul_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int32_t, int32_t, void *stream) {
    return csr2_run<OP_INTERSECT>(a, b, z, true, 0, stream);
}

int nb200_csr_mul_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream) {
    return csr2_run<OP_INTERSECT>(a, b, z, false, capacity, stream);
}

}  // extern "C"
