// Host-buffer entry points for CSR add / multiply: operands and result live in host memory and
// are streamed through the GPU in row blocks, so that the host-to-device copy of block k+1,
// the merge of block k and the device-to-host copy of block k-1 run at the same time (PCIe
// is full duplex). Rows are independent, so the blocks need nothing from each other except
// the running result length, which is added to each block's row offsets on the device.
//
// The reference has no such call (its operators take device tensors); this is the form of the
// same operator for callers whose data starts and ends on the host.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace nb200 {

namespace {

constexpr int SLOTS = 3;                      // block k+1 loading, k merging, k-1 draining
constexpr int64_t BLOCK_ENTRIES = 12 << 20;   // operand entries per block (A + B) unless NACHO_B200_HOST_BLOCK names another count

int64_t block_entries() {
    static const int64_t n = [] {
        const char *e = std::getenv("NACHO_B200_HOST_BLOCK");
        const long long v = e ? std::atoll(e) : 0;
        return v >= 1024 ? (int64_t)v : BLOCK_ENTRIES;
    }();
    return n;
}

struct Pipeline {
    cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
    cudaEvent_t loaded[SLOTS] = {}, merged[SLOTS] = {}, drained[SLOTS] = {}, counted[SLOTS] = {};
    // Result words of a block's merge (length, status, rows), four per slot, in pinned host memory
    // the GPU writes straight into: a length read back with a copy would queue behind the previous
    // block's device-to-host copy on the copy engine.
    int64_t *words = nullptr;
    bool ready = false;
    std::mutex busy;  // held for a whole call: the streams, events and device buffers serve one call at a time
};

std::mutex g_pipe_mutex;
Pipeline g_pipes[64];

int get_pipeline(Pipeline **out) {
    int dev = 0;
    NB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NB200_E_UNSUPPORTED;
    std::lock_guard<std::mutex> g(g_pipe_mutex);
    Pipeline &p = g_pipes[dev];
    if (!p.ready) {
        NB200_CUDA(cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking));
        NB200_CUDA(cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking));
        NB200_CUDA(cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking));
        for (int s = 0; s < SLOTS; ++s) {
            NB200_CUDA(cudaEventCreateWithFlags(&p.loaded[s], cudaEventDisableTiming));
            NB200_CUDA(cudaEventCreateWithFlags(&p.merged[s], cudaEventDisableTiming));
            NB200_CUDA(cudaEventCreateWithFlags(&p.drained[s], cudaEventDisableTiming));
            NB200_CUDA(cudaEventCreateWithFlags(&p.counted[s], cudaEventDisableTiming));
        }
        NB200_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&p.words), sizeof(int64_t) * 4 * SLOTS, cudaHostAllocMapped));
        p.ready = true;
    }
    *out = &p;
    return NB200_OK;
}

__global__ void __launch_bounds__(256) k_add_base(int32_t *rp, int32_t n, int32_t base) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) rp[i] += base;
}

struct Block {
    int32_t r0, r1;      // rows [r0, r1)
    int64_t a0, a1, b0, b1;  // entry ranges of A and B
};

// Device arrays of one pipeline slot.
struct SlotArrays {
    int32_t *a_rp, *b_rp, *a_col, *b_col, *z_rp, *z_col;
    float *a_val, *b_val, *z_val;
};

typedef int (*into_fn)(const nb200_csr *, const nb200_csr *, nb200_csr *, int64_t, int64_t *, void *);  // the asynchronous form

int csr2_host_locked(Pipeline *pipe, into_fn op, bool is_union, const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity);

// Validates, takes the device's pipeline for the whole call (concurrent callers on one device queue
// up here), runs, and on any failure waits for every copy already queued on the three streams:
// those copies read and write the caller's host buffers, which the caller may release as soon as
// the call has returned.
int csr2_host(into_fn op, bool is_union, const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity) {
    if (!a || !b || !z || a->rows != b->rows || a->cols != b->cols || a->rows < 0 || capacity < 0) return NB200_E_BADARG;
    if (!a->row_ptr || !b->row_ptr || !z->row_ptr) return NB200_E_BADARG;
    Pipeline *pipe = nullptr;
    int st;
    if ((st = get_pipeline(&pipe))) return st;
    std::lock_guard<std::mutex> busy(pipe->busy);
    st = csr2_host_locked(pipe, op, is_union, a, b, z, capacity);
    if (st != NB200_OK) {
        cudaStreamSynchronize(pipe->in);
        cudaStreamSynchronize(pipe->compute);
        cudaStreamSynchronize(pipe->out);
        cudaGetLastError();
    }
    return st;
}

int csr2_host_locked(Pipeline *pipe, into_fn op, bool is_union, const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity) {
    if (!a || !b || !z || a->rows != b->rows || a->cols != b->cols || a->rows < 0 || capacity < 0) return NB200_E_BADARG;
    if (!a->row_ptr || !b->row_ptr || !z->row_ptr) return NB200_E_BADARG;
    const int32_t rows = a->rows;
    const int32_t *arp = a->row_ptr, *brp = b->row_ptr;
    z->rows = rows;
    z->cols = a->cols;
    z->nnz = 0;
    z->row_ptr[0] = 0;
    if (rows == 0) return NB200_OK;

    // ---- row blocks of about block_entries() operand entries
    std::vector<Block> blocks;
    int64_t max_a = 0, max_b = 0;
    int32_t max_rows = 0;
    for (int32_t r = 0; r < rows;) {
        int32_t e = r;
        const int64_t start = (int64_t)arp[r] + brp[r];
        while (e < rows && ((int64_t)arp[e + 1] + brp[e + 1]) - start <= block_entries()) ++e;
        if (e == r) e = r + 1;  // a single row larger than a block still goes through whole
        Block blk{r, e, arp[r], arp[e], brp[r], brp[e]};
        blocks.push_back(blk);
        max_a = std::max(max_a, blk.a1 - blk.a0);
        max_b = std::max(max_b, blk.b1 - blk.b0);
        max_rows = std::max(max_rows, e - r);
        r = e;
    }
    const int64_t max_z = is_union ? max_a + max_b : std::min(max_a, max_b);

    int st;
    Carver sizes;
    for (int s = 0; s < SLOTS; ++s) {
        for (int q = 0; q < 3; ++q) sizes.take<int32_t>((size_t)max_rows + 1);
        sizes.take<int32_t>((size_t)max_a), sizes.take<float>((size_t)max_a);
        sizes.take<int32_t>((size_t)max_b), sizes.take<float>((size_t)max_b);
        sizes.take<int32_t>((size_t)max_z), sizes.take<float>((size_t)max_z);
    }
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(pipe->compute, sizes.used(), &ws, 2))) return st;
    Carver carve(ws->dev);
    SlotArrays slot[SLOTS];
    for (int s = 0; s < SLOTS; ++s) {
        slot[s].a_rp = carve.take<int32_t>((size_t)max_rows + 1);
        slot[s].b_rp = carve.take<int32_t>((size_t)max_rows + 1);
        slot[s].z_rp = carve.take<int32_t>((size_t)max_rows + 1);
        slot[s].a_col = carve.take<int32_t>((size_t)max_a), slot[s].a_val = carve.take<float>((size_t)max_a);
        slot[s].b_col = carve.take<int32_t>((size_t)max_b), slot[s].b_val = carve.take<float>((size_t)max_b);
        slot[s].z_col = carve.take<int32_t>((size_t)max_z), slot[s].z_val = carve.take<float>((size_t)max_z);
    }

    auto load = [&](int k) -> int {
        const Block &blk = blocks[k];
        const SlotArrays &d = slot[k % SLOTS];
        if (k >= SLOTS) NB200_CUDA(cudaStreamWaitEvent(pipe->in, pipe->drained[k % SLOTS], 0));
        const size_t nr = (size_t)(blk.r1 - blk.r0) + 1, na = (size_t)(blk.a1 - blk.a0), nb = (size_t)(blk.b1 - blk.b0);
        NB200_CUDA(cudaMemcpyAsync(d.a_rp, arp + blk.r0, 4 * nr, cudaMemcpyHostToDevice, pipe->in));
        NB200_CUDA(cudaMemcpyAsync(d.b_rp, brp + blk.r0, 4 * nr, cudaMemcpyHostToDevice, pipe->in));
        if (na) {
            NB200_CUDA(cudaMemcpyAsync(d.a_col, a->col + blk.a0, 4 * na, cudaMemcpyHostToDevice, pipe->in));
            NB200_CUDA(cudaMemcpyAsync(d.a_val, a->val + blk.a0, 4 * na, cudaMemcpyHostToDevice, pipe->in));
        }
        if (nb) {
            NB200_CUDA(cudaMemcpyAsync(d.b_col, b->col + blk.b0, 4 * nb, cudaMemcpyHostToDevice, pipe->in));
            NB200_CUDA(cudaMemcpyAsync(d.b_val, b->val + blk.b0, 4 * nb, cudaMemcpyHostToDevice, pipe->in));
        }
        NB200_CUDA(cudaEventRecord(pipe->loaded[k % SLOTS], pipe->in));
        return NB200_OK;
    };

    int64_t produced = 0;
    if ((st = load(0))) return st;
    for (int k = 0; k < (int)blocks.size(); ++k) {
        if (k + 1 < (int)blocks.size() && (st = load(k + 1))) return st;
        const Block &blk = blocks[k];
        const SlotArrays &d = slot[k % SLOTS];
        NB200_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->loaded[k % SLOTS], 0));
        // the block's row offsets keep their absolute values; the column / value pointers are
        // shifted so that those absolute positions land inside the block's arrays
        nb200_csr va{blk.r1 - blk.r0, a->cols, (int32_t)(blk.a1 - blk.a0), d.a_rp, d.a_col - blk.a0, d.a_val - blk.a0};
        nb200_csr vb{blk.r1 - blk.r0, b->cols, (int32_t)(blk.b1 - blk.b0), d.b_rp, d.b_col - blk.b0, d.b_val - blk.b0};
        nb200_csr vz{0, 0, 0, d.z_rp, d.z_col, d.z_val};
        volatile int64_t *words = pipe->words + 4 * (k % SLOTS);
        int64_t *words_dev = nullptr;
        NB200_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&words_dev), pipe->words + 4 * (k % SLOTS), 0));
        if ((st = op(&va, &vb, &vz, max_z, words_dev, pipe->compute))) return st;
        NB200_CUDA(cudaEventRecord(pipe->counted[k % SLOTS], pipe->compute));
        NB200_CUDA(cudaEventSynchronize(pipe->counted[k % SLOTS]));  // the block's length is known
        if (words[1] != NB200_OK) return (int)words[1];
        const int64_t n = words[0];
        if (produced + n > capacity || produced + n > INT32_MAX) {  // the caller drains the streams
            z->nnz = (int32_t)std::min<int64_t>(produced + n, INT32_MAX);
            return produced + n > INT32_MAX ? NB200_E_OVERFLOW : NB200_E_CAPACITY;
        }
        const int nr = blk.r1 - blk.r0;
        if (produced) k_add_base<<<(nr + 256) / 256, 256, 0, pipe->compute>>>(d.z_rp, nr + 1, (int32_t)produced);
        NB200_CUDA(cudaEventRecord(pipe->merged[k % SLOTS], pipe->compute));
        NB200_CUDA(cudaStreamWaitEvent(pipe->out, pipe->merged[k % SLOTS], 0));
        NB200_CUDA(cudaMemcpyAsync(z->row_ptr + blk.r0 + 1, d.z_rp + 1, 4 * (size_t)nr, cudaMemcpyDeviceToHost, pipe->out));
        if (n) {
            NB200_CUDA(cudaMemcpyAsync(z->col + produced, d.z_col, 4 * (size_t)n, cudaMemcpyDeviceToHost, pipe->out));
            NB200_CUDA(cudaMemcpyAsync(z->val + produced, d.z_val, 4 * (size_t)n, cudaMemcpyDeviceToHost, pipe->out));
        }
        NB200_CUDA(cudaEventRecord(pipe->drained[k % SLOTS], pipe->out));
        produced += n;
    }
    NB200_CUDA(cudaStreamSynchronize(pipe->out));
    z->nnz = (int32_t)produced;
    return NB200_OK;
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_csr_add_f32_host(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity) {
    return csr2_host(nb200_csr_add_f32_async, true, a, b, z, capacity);
}

int nb200_csr_mul_f32_host(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity) {
    return csr2_host(nb200_csr_mul_f32_async, false, a, b, z, capacity);
}

}  // extern "C"
