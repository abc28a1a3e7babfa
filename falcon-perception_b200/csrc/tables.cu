// The allocator's device side: free-page stack, free-slot stack and the two page tables.
//
// The reference keeps its free lists in Python and, for every allocate / reserve / erase call,
// updates the device tables with a few tiny tensor operations plus one host-to-device tensor
// (falcon_perception/paged_attention.py:102-109, 145-158, 166-182); erase and allocate rewrite
// both table rows of the slot in full (2 x n_pages entries).  Here the free lists live on the
// device as stacks laid out like the reference's lists (bottom first, the list's last element
// on top), and one launch applies a whole scheduling step's calls: the host sends one 16-byte
// record per call -- not per page -- and keeps its own mirror of the lists, which it needs for
// can_reserve and the error text anyway.
//
// Records are applied in order.  The order only matters along three chains: the slot stack
// (erase pushes, allocate pops), the page stack (erase pushes what a later reserve pops), and
// the table rows of one slot.  So thread 0 first walks the records once, doing the slot stack
// and working out where on the page stack every record starts; then runs of consecutive
// records of the same kind execute in parallel, one warp per record, lanes over its pages,
// with a CTA barrier between runs.  An erase touches only the entries the slot owns.

#include "common.cuh"

namespace fpkv {

namespace {

constexpr int kAllocThreads = 512;
constexpr int kAllocWarps = kAllocThreads / 32;
constexpr int kMaxOpsPerLaunch = 2048;

enum : int { kOpAllocate = 0, kOpReserve = 1, kOpErase = 2, kOpMap = 3, kOpClear = 4 };

__global__ void __launch_bounds__(kAllocThreads)
alloc_step_kernel(int64_t* __restrict__ page_table, int64_t* __restrict__ p2l, int n_pages, int max_batch,
                  int32_t* __restrict__ free_pages, int32_t* __restrict__ free_slots, int32_t* __restrict__ counts,
                  const int4* __restrict__ ops, int n_ops, int32_t* status)
{
    __shared__ int4 s_op[kMaxOpsPerLaunch];
    __shared__ int s_base[kMaxOpsPerLaunch];           // page-stack height before the record; -1 = record skipped
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    for (int i = tid; i < n_ops; i += kAllocThreads) s_op[i] = ops[i];
    __syncthreads();

    // ---- pass 1 (one thread): slot stack, page-stack offsets, argument checks ------------
    if (tid == 0) {
        int np = counts[0], ns = counts[1];
        for (int i = 0; i < n_ops; ++i) {
            const int4 op = s_op[i];
            int base = -1;
            if (op.y <= 0 || op.y >= max_batch) {          // slot 0 is the reserved no-op slot: never edited
                raise_status(status, FPKV_STATUS_BAD_SLOT);
            } else if (op.x == kOpAllocate) {              // pop; the host's mirror said which slot this must be
                if (ns <= 0 || free_slots[ns - 1] != op.y) raise_status(status, FPKV_STATUS_BAD_SLOT);
                else --ns;
            } else if (op.x == kOpReserve) {               // a = first logical page, b = pages to take
                if (op.w < 0 || op.w > np || op.z < 0 || op.z + op.w > n_pages) raise_status(status, FPKV_STATUS_BAD_PAGE);
                else { np -= op.w; base = np; }            // takes stack[np - n, np) in list order
            } else if (op.x == kOpErase) {                 // a = pages the slot owns (logical 0 .. a-1)
                if (op.z < 0 || op.z > n_pages || np + op.z > n_pages || ns >= max_batch) raise_status(status, FPKV_STATUS_BAD_PAGE);
                else { base = np; np += op.z; free_slots[ns++] = op.y; }
            } else if (op.x == kOpMap) {                   // a = logical page, b = physical page (page 0 is reserved)
                if (op.z < 0 || op.z >= n_pages || op.w <= 0 || op.w >= n_pages) raise_status(status, FPKV_STATUS_BAD_PAGE);
                else base = 0;
            } else if (op.x == kOpClear) {
                base = 0;
            } else {
                raise_status(status, FPKV_STATUS_BAD_SLOT);
            }
            s_base[i] = base;
        }
        counts[0] = np; counts[1] = ns;
    }
    __syncthreads();

    // ---- pass 2: runs of equal kind in parallel, one warp per record ---------------------
    int i0 = 0;
    while (i0 < n_ops) {
        int k = i0;
        while (k < n_ops && s_op[k].x == kOpAllocate) ++k;     // allocate has no table work
        if (k == n_ops) break;
        const int kind = s_op[k].x;
        int i1 = k + 1;
        if (kind == kOpReserve || kind == kOpErase)
            while (i1 < n_ops && (s_op[i1].x == kind || s_op[i1].x == kOpAllocate)) ++i1;
        if (kind == kOpClear) {                                // both rows in full, all threads
            if (s_base[k] >= 0) {
                int64_t* pt = page_table + (size_t)s_op[k].y * n_pages;
                int64_t* il = p2l + (size_t)s_op[k].y * n_pages;
                for (int j = tid; j < n_pages; j += kAllocThreads) { pt[j] = -1; il[j] = -1; }
            }
        } else {
            for (int i = k + warp; i < i1; i += kAllocWarps) {
                const int4 op = s_op[i];
                const int base = s_base[i];
                if (base < 0 || op.x == kOpAllocate) continue;
                int64_t* pt = page_table + (size_t)op.y * n_pages;
                int64_t* il = p2l + (size_t)op.y * n_pages;
                if (op.x == kOpReserve) {
                    for (int j = lane; j < op.w; j += 32) {
                        const int pg = free_pages[base + j];
                        if (pg <= 0 || pg >= n_pages) { raise_status(status, FPKV_STATUS_BAD_PAGE); continue; }
                        pt[op.z + j] = pg; il[pg] = op.z + j;
                    }
                } else if (op.x == kOpErase) {                 // free_pages.extend(reversed(pages)); entries back to -1
                    for (int j = lane; j < op.z; j += 32) {
                        const long long pg = pt[j];
                        free_pages[base + (op.z - 1 - j)] = (int)pg;
                        pt[j] = -1;
                        if (pg > 0 && pg < n_pages) il[pg] = -1; else raise_status(status, FPKV_STATUS_BAD_PAGE);
                    }
                } else if (lane == 0) {                        // kOpMap
                    pt[op.z] = op.w; il[op.w] = op.z;
                }
            }
        }
        __syncthreads();                                       // the next run may read what this one wrote
        i0 = i1;
    }
}

}  // namespace

int launch_alloc_step(int64_t* page_table, int64_t* p2l, int n_pages, int max_batch, int32_t* free_pages,
                      int32_t* free_slots, int32_t* counts, const int32_t* ops, int n_ops, int32_t* status,
                      cudaStream_t stream)
{
    for (int at = 0; at < n_ops; at += kMaxOpsPerLaunch) {
        const int n = n_ops - at < kMaxOpsPerLaunch ? n_ops - at : kMaxOpsPerLaunch;
        alloc_step_kernel<<<1, kAllocThreads, 0, stream>>>(page_table, p2l, n_pages, max_batch, free_pages, free_slots,
                                                           counts, reinterpret_cast<const int4*>(ops) + at, n, status);
        if (cudaGetLastError() != cudaSuccess) return FPKV_ELAUNCH;
    }
    return FPKV_OK;
}

}  // namespace fpkv
