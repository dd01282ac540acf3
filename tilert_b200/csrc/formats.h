// Packed data formats shared by the host packers and the kernels.
//
// Weight block ("W block"): one 128-row x 128-column e4m3 tile of a weight matrix plus its
// dequantisation scales, laid out so that one bulk copy brings a whole pipeline stage into
// shared memory in the form the tensor core reads through a shared-memory descriptor (K-major,
// no swizzle: 8-row x 16-byte "core matrices" of 128 contiguous bytes):
//
//   byte c*4096 + (row/8)*256 + kc*128 + (row%8)*16 + b   holds   W[row, 32*c + 16*kc + b]
//   for k chunk c in 0..3 (one MMA each), core column kc in 0..1, b in 0..15;
//   bytes 16384 .. 16447: 16 f32 scales, one per group of 8 consecutive packed rows.
//
// A matrix [N, K] is stored as blocks in (row tile, k block) order, the k blocks of one
// row tile being contiguous.  Packed rows may be any permutation of the source rows as long
// as each aligned group of 8 packed rows shares one source scale.
//
// Activation block ("X block"): the 128 activations of one k block for up to 8 columns
// (tokens, or hi/lo halves of tokens) in the same core-matrix form, plus one f32 scale per column:
//
//   byte c*256 + kc*128 + col*16 + b   holds   X[col, k = 32*c + 16*kc + b]
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
