// The tiled unit layout, in one place.  unit_offset(type, i, raw_off) maps byte `raw_off` of the
// GGUF bytes that hold row i's 256-weight segment (8 x 18 B for Q4_0, 8 x 34 B for Q8_0, one
// 144 B super-block for Q4_K, one 210 B super-block for Q6_K; block layouts as decoded in
// crates/tl_runtime/src/quantized.rs:182-415) to its byte offset inside the 16-row unit.
//
// Lane (r, c) = (lane/4, lane%4) of the consuming warp owns rows r and r+8 (hi = 0 / 1) of the tile
// and, in the A fragment of mma.m16n8k32 (8-bit operands), the k positions 4c..4c+3 (h = 0) and
// 16+4c..16+4c+3 (h = 1) of every block of 32.  Quant bytes sit in 16-byte pieces at
// piece*512 + lane*16, one 32-bit word (4 consecutive k) per slot, so every shared-memory read of
// the matvec kernel is a conflict-free 128-bit load that lands directly in MMA operand order.
#pragma once
#include <cstdint>

namespace tlb {

__host__ __device__ inline int unit_offset(int type, int i, int raw_off)
{
    const int r = i & 7, hi = i >> 3;
    if (type == 12) {  // Q4_K: [d, dmin, scales[12]] [qs[128]]
        // group G = 32 bytes: low nibbles are sub-block 2G (k = 64G + l), high nibbles sub-block 2G+1
        if (raw_off < 16) return 2048 + i * 16 + raw_off;
        int qb = raw_off - 16, G = qb >> 5, within = qb & 31;
        int h = within >> 4, c = (within & 15) >> 2, byte = within & 3;
        return G * 512 + (r * 4 + c) * 16 + (hi * 2 + h) * 4 + byte;
    }
    if (type == 2) {  // Q4_0: 8 x [d][qs[16]]; byte j: low nibble k = j, high nibble k = 16 + j
        int b = raw_off / 18, o = raw_off % 18;
        if (o < 2) return 2048 + i * 16 + b * 2 + o;
        int qb = o - 2, c = qb >> 2, byte = qb & 3;
        int piece = b >> 1, slot = hi * 2 + (b & 1);
        return piece * 512 + (r * 4 + c) * 16 + slot * 4 + byte;
    }
    if (type == 8) {  // Q8_0: 8 x [d][q[32]]
        int b = raw_off / 34, o = raw_off % 34;
        if (o < 2) return 4096 + i * 16 + b * 2 + o;
        int qb = o - 2, j = qb >> 2, byte = qb & 3;  // word j covers k = 4j..4j+3
        int c = j & 3, h = j >> 2;
        int slot = hi * 2 + h;
        return b * 512 + (r * 4 + c) * 16 + slot * 4 + byte;
    }
    // Q6_K: ql[128] qh[64] scales[16] d
    if (raw_off < 128) {
        int n = raw_off >> 6, w = raw_off & 63, q1 = w >> 5, l = w & 31;
        int h = l >> 4, c = (l & 15) >> 2, byte = l & 3;
        int piece = hi * 2 + n, slot = q1 * 2 + h;
        return piece * 512 + (r * 4 + c) * 16 + slot * 4 + byte;
    }
    if (raw_off < 192) {
        int hh = raw_off - 128, n = hh >> 5, l = hh & 31;
        int h = l >> 4, c = (l & 15) >> 2, byte = l & 3;
        int slot = n * 2 + h;
        return 2048 + hi * 512 + (r * 4 + c) * 16 + slot * 4 + byte;
    }
    if (raw_off < 208) return 3072 + i * 16 + (raw_off - 192);
    return 3328 + i * 2 + (raw_off - 208);
}

}  // namespace tlb
