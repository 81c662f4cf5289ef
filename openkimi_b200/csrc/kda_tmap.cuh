// Tensor maps for the token-major BF16 tensors [tokens][H][128] (q, k, v, g, o and their gradients): the 64 rows
// that one (chunk, head) unit reads or writes are 256 bytes each and H * 256 bytes apart, so a tiled bulk-tensor
// copy moves the whole [64 x 128] tile with one instruction where 64 separate row copies would queue up in the
// copy unit.  The maps are encoded on the host at every call (they hold the caller's pointers) and travel as
// kernel parameters.
#pragma once
#include <cuda.h>

#include "kda_common.cuh"
#include "kda_tc.cuh"

namespace kda {

struct RowMaps {
    CUtensorMap m[4];
    int ok;  // 0: the driver's encoder is not available; the kernels then copy row by row
};

// [tokens][H * 128] BF16 at base, box = [box_rows][128]; false when the encoder is missing or refuses
bool make_row_map(CUtensorMap* out, const void* base, long long tokens, int H, int box_rows);

namespace tc {
// tile (rows y .. y + box_rows - 1, elements x .. x + 127) -> shared memory (dense, row-major); x * 2 bytes
// must be a multiple of 16 (x = 128 * head always is)
__device__ __forceinline__ void tma_load_tile(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// shared memory (dense, row-major) -> tile; y must not be negative
__device__ __forceinline__ void tma_store_tile(const CUtensorMap* map, int x, int y, const void* src_smem) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
                 "r"(smem_u32(src_smem))
                 : "memory");
}
}  // namespace tc
}  // namespace kda
