// Packed data formats shared by the host packers and the kernels.
//
// Weight block ("W block"): one 128-row x 128-column e4m3 tile of a weight matrix plus its
// dequantisation scales, laid out so that one bulk copy brings a whole pipeline stage into
// shared memory and every warp reads its m16n8k32 A fragments with one conflict-free 16-byte
// load per lane:
//
//   byte ((w*4 + c)*32 + lane)*16 + 4*r + b   holds   W[row, col]   with
//       row = 16*w + (lane/4) + 8*(r&1),   col = 32*c + 16*(r>>1) + 4*(lane%4) + b
//   for warp w in 0..7 (16 rows each), k-chunk c in 0..3, register r in 0..3, byte b in 0..3;
//   bytes 16384 .. 16447: 16 f32 scales, one per group of 8 consecutive packed rows.
//
// A matrix [N, K] is stored as blocks in (row tile, k block) order, the k blocks of one
// row tile being contiguous.  Packed rows may be any permutation of the source rows as long
// as each aligned group of 8 packed rows shares one source scale.
//
// Activation block ("X block"): the 128 activations of one k block for up to 8 columns
// (tokens, or hi/lo halves of tokens), in m16n8k32 B-fragment order, plus one f32 scale per
// column:
//
//   byte (c*32 + lane)*8 + 4*r + b   holds   X[col = lane/4, k = 32*c + 16*r + 4*(lane%4) + b]
//   bytes 1024 .. 1055: 8 f32 column scales.
//
// In "split" mode column 2t holds the leading e4m3 term of token t and column 2t+1 the e4m3
// residual term, so that hi*s_hi + lo*s_lo reproduces a bf16 activation exactly.
#pragma once

#define TB_TILE_ROWS 128
#define TB_KBLOCK 128
#define TB_WBLK_DATA 16384
#define TB_WBLK_BYTES 16448
#define TB_XBLK_DATA 1024
#define TB_XBLK_BYTES 1056
#define TB_STAGE_BYTES (TB_WBLK_BYTES + TB_XBLK_BYTES)
#define TB_MAX_REGIONS 4
