// Page-table maintenance on the device.
//
// The reference updates its device tables with a few tiny tensor operations and
// one host-to-device tensor per allocate / reserve / erase call
// (falcon_perception/paged_attention.py:102-109, 145-158, 166-182).  Here the
// host keeps doing the bookkeeping (free lists, capacities: it needs them for
// can_reserve anyway) and queues the table edits; one launch applies a whole
// step's worth of them in order.

#include "common.cuh"

namespace fpkv {

// ops[i] = {kind, slot, a, b}
//   kind 0  clear: page_table[slot, :] = physical_to_logical[slot, :] = -1      (allocate, erase)
//   kind 1  map:   page_table[slot, a] = b; physical_to_logical[slot, b] = a    (reserve)
// Edits are applied in order (a slot may be cleared and mapped again in one batch).
__global__ void __launch_bounds__(256)
table_update_kernel(int64_t* __restrict__ page_table, int64_t* __restrict__ p2l, int n_pages, int max_batch,
                    const int4* __restrict__ ops, int n_ops, int32_t* status)
{
    for (int i = 0; i < n_ops; ++i) {
        const int4 op = ops[i];
        if (op.y <= 0 || op.y >= max_batch) {              // slot 0 is the reserved no-op slot: never edited
            if (threadIdx.x == 0) raise_status(status, FPKV_STATUS_BAD_SLOT);
            continue;
        }
        int64_t* pt = page_table + (size_t)op.y * n_pages;
        int64_t* il = p2l + (size_t)op.y * n_pages;
        if (op.x == 0) {
            for (int j = threadIdx.x; j < n_pages; j += blockDim.x) { pt[j] = -1; il[j] = -1; }
        } else if (threadIdx.x == 0) {
            if (op.z < 0 || op.z >= n_pages || op.w <= 0 || op.w >= n_pages) raise_status(status, FPKV_STATUS_BAD_PAGE);
            else { pt[op.z] = op.w; il[op.w] = op.z; }
        }
        __syncthreads();                                   // the next edit may touch the same row
    }
}

int launch_table_update(int64_t* page_table, int64_t* p2l, int n_pages, int max_batch, const int32_t* ops,
                        int n_ops, int32_t* status, cudaStream_t stream)
{
    if (n_ops == 0) return FPKV_OK;
    table_update_kernel<<<1, 256, 0, stream>>>(page_table, p2l, n_pages, max_batch,
                                               reinterpret_cast<const int4*>(ops), n_ops, status);
    return cudaGetLastError() == cudaSuccess ? FPKV_OK : FPKV_ELAUNCH;
}

}  // namespace fpkv
