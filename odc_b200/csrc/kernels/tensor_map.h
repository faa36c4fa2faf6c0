// Host helper: build TMA tensor maps (bf16, 128-byte swizzle, zero fill outside the tensor).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace odc {

// 2-D row-major bf16 tensor [outer, inner] with `row_pitch_bytes` between rows; tiles of
// box_inner x box_outer elements.  Returns false if the driver rejects the description.
bool encode_tile_map_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                        uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// 2-D row-major fp32 tensor, tiles of box_inner x box_outer elements (box_inner * 4 bytes == 128 for the swizzle).
bool encode_tile_map_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                            uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer);

// 3-D bf16 tensor [d2, d1, d0] (d0 innermost, contiguous) with byte pitches for d1 and d2.
bool encode_tile_map_3d(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0, uint32_t box1, uint32_t box2);

// Make `device`'s primary context current for the calling thread in this library's CUDA runtime.
// Threads created by PyTorch's autograd engine may not have a driver context bound yet, and
// tensor-map encoding is a driver call that needs one.
void bind_device(int device);

}  // namespace odc
