// Compiled kernel configurations.
//
// Variant ids.  In every argument block `variant` 0 means "let the library choose" (by head size,
// and by how the grid of sequences fills the GPU); every compiled configuration also has an explicit
// id >= 1 that is always honoured, so that configurations can be timed against each other through
// the same ABI.  The ids of one (operator, head size) are contiguous from 1.  The configurations the
// automatic choice can pick are always compiled; the remaining ones are tuning alternatives and are
// compiled only with -DSRWM_TUNING_VARIANTS (csrc/build.py --tuning).
//
// Register-tile kernels: X(E, id, P, R, T, PK, MINB, LAYER)
//   E      head dimension            P     threads per sequence (= CTA size)
//   R      state rows per thread     T     time steps staged per chunk
//   PK     packed fma.rn.f32x2 (1) or scalar fma (0)
//   MINB   CTAs per SM the register allocation is bounded for (__launch_bounds__)
//   LAYER  1: the layer-level form of the call (input softmax, base + shift state, reset flags;
//          packed rows for the delta rule) is instantiated for this configuration too
#pragma once

#ifdef SRWM_TUNING_VARIANTS
#define SRWM_TUNING(...) __VA_ARGS__
#else
#define SRWM_TUNING(...)
#endif

// ---- SRWM forward -------------------------------------------------------------------------------
// Automatic choice: E = 8, 16 register tiles (id 1); E = 64 column layout (id 1); E = 32 column layout
// (id 1) up to eight sequences per multiprocessor, one warp per sequence (id 2) beyond (measured, 1776
// sequences x 512 steps: 0.71 against 0.92 ms; 256 sequences x 100 steps: 0.137 against 0.126 ms).
#define SRWM_FWD_CONFIGS(X)              \
  X(8, 1, 32, 2, 16, true, 8, 1)         \
  X(16, 1, 32, 4, 16, true, 8, 1)        \
  SRWM_TUNING(                           \
  X(16, 2, 32, 2, 16, true, 8, 0)        \
  X(32, 3, 64, 8, 16, true, 6, 0)        \
  X(32, 4, 32, 8, 16, true, 8, 0)        \
  X(32, 5, 64, 4, 16, true, 6, 0)        \
  X(64, 2, 128, 8, 16, true, 3, 0)       \
  X(64, 3, 128, 16, 16, true, 3, 0)      \
  X(64, 4, 128, 8, 16, false, 3, 0))

// Column-layout forward (96 threads, one warp per block): Y(E, id, T, PK, MINB, DPRE, NRP, LAYER)
//   DPRE  the k warp publishes q-k once per step (two-warp named barrier) instead of every
//         thread recomputing it in the second pass
//   NRP   row parts per column group (1 = whole columns per lane)
#define SRWM_FWD_COL_CONFIGS(Y)          \
  Y(32, 1, 16, true, 8, true, 2, 1)      \
  Y(64, 1, 16, true, 4, true, 1, 1)      \
  SRWM_TUNING(                           \
  Y(16, 3, 16, true, 8, true, 2, 0)      \
  Y(16, 4, 16, true, 16, true, 2, 0)     \
  Y(32, 6, 16, true, 8, false, 1, 0)     \
  Y(32, 7, 16, true, 8, true, 1, 0)      \
  Y(32, 8, 16, true, 8, true, 4, 0)      \
  Y(32, 9, 16, true, 12, true, 4, 0)     \
  Y(64, 5, 16, true, 4, false, 1, 0)     \
  Y(64, 6, 16, true, 4, true, 2, 0)      \
  Y(64, 7, 16, true, 4, true, 4, 0)      \
  Y(64, 8, 16, false, 4, true, 2, 0)     \
  Y(64, 9, 16, true, 3, true, 2, 0))

// E lanes per sequence, 32 / E sequences per warp (srwm_fwd_warp.cuh, head sizes up to 32): V(E, id, T, MINB), T <= E;
// serves the layer-level form too
#define SRWM_FWD_WARP_CONFIGS(V)         \
  V(32, 2, 16, 12)                       \
  SRWM_TUNING(                           \
  V(8, 2, 8, 24)                         \
  V(16, 5, 16, 16)                       \
  V(32, 10, 8, 12))

// ---- SRWM backward ------------------------------------------------------------------------------
#define SRWM_BWD_CONFIGS(X)              \
  X(8, 1, 32, 2, 16, true, 8, 1)         \
  X(16, 1, 32, 2, 16, true, 8, 1)        \
  X(32, 1, 64, 4, 16, true, 6, 1)        \
  SRWM_TUNING(                           \
  X(16, 2, 32, 4, 16, true, 8, 0)        \
  X(32, 2, 64, 8, 16, true, 6, 0)        \
  X(32, 3, 32, 8, 16, true, 8, 0)        \
  X(64, 2, 128, 8, 16, true, 2, 1)       \
  X(64, 3, 256, 8, 16, true, 1, 0)       \
  X(64, 4, 128, 8, 16, false, 2, 0))

// Second formulation of the backward (srwm_bwd2.cuh): Z(E, id, P, R, T, MINB, OPT); always serves the
// layer-level form as well
#define SRWM_BWD2_CONFIGS(Z)             \
  Z(64, 1, 128, 8, 16, 2, 4)             \
  SRWM_TUNING(                           \
  Z(32, 4, 64, 4, 16, 5, 0)              \
  Z(32, 5, 64, 4, 8, 6, 0)               \
  Z(64, 5, 128, 8, 16, 2, 0)             \
  Z(64, 6, 128, 8, 16, 2, 6)             \
  Z(64, 7, 128, 8, 16, 2, 12))

// Backward with the state detached at every step (W_y and its gradient only): X(E, id, P, R, T, PK, MINB)
#define SRWM_BWD_DET_CONFIGS(X)          \
  X(8, 1, 32, 2, 16, true, 8)            \
  X(16, 1, 32, 4, 16, true, 8)           \
  X(32, 1, 64, 8, 16, true, 6)           \
  X(64, 1, 128, 16, 16, true, 4)

// ---- delta rule forward -------------------------------------------------------------------------
// At E = 64 the automatic choice is the column kernel: id 1 (one warp per sequence) when the grid fills
// the GPU, id 3 (four warps per sequence) when there are so few sequences that a lone warp's step
// latency is exposed; the packed (layer-level) form uses id 1 / id 4.
#define DELTA_FWD_CONFIGS(X)             \
  X(8, 1, 32, 2, 16, true, 8, 1)         \
  X(16, 1, 32, 4, 16, true, 8, 1)        \
  X(32, 1, 32, 8, 16, true, 12, 1)       \
  X(64, 4, 64, 16, 8, true, 8, 1)        \
  SRWM_TUNING(                           \
  X(32, 2, 64, 8, 16, true, 8, 0)        \
  X(64, 5, 64, 32, 8, true, 8, 0)        \
  X(64, 6, 64, 64, 8, true, 8, 0)        \
  X(64, 7, 128, 16, 8, true, 6, 0)       \
  X(64, 8, 32, 16, 8, true, 10, 0)       \
  X(64, 9, 64, 16, 8, false, 8, 0))

// Column-layout delta forward: Y(E, id, P, T, PK, MINB, NRP, LAYER, UNR)   UNR: unrolling of the step loop
#define DELTA_FWD_COL_CONFIGS(Y)         \
  Y(64, 1, 32, 8, true, 8, 1, 1, 1)      \
  Y(64, 2, 64, 8, true, 7, 2, 0, 1)      \
  Y(64, 3, 128, 16, true, 4, 2, 0, 2)    \
  SRWM_TUNING(                           \
  Y(32, 3, 32, 16, true, 16, 1, 0, 1)    \
  Y(32, 4, 32, 16, true, 16, 2, 0, 1)    \
  Y(64, 10, 32, 8, true, 8, 2, 0, 1)     \
  Y(64, 11, 64, 8, true, 8, 1, 0, 1)     \
  Y(64, 12, 128, 8, true, 4, 2, 0, 1)    \
  Y(64, 13, 128, 32, true, 3, 2, 0, 2))

// ---- delta rule backward ------------------------------------------------------------------------
// At E = 64: id 1 (64 threads per sequence) on whole waves; id 2 (128) for the sequences of a partial
// last wave and for small grids.
#define DELTA_BWD_CONFIGS(X)             \
  X(8, 1, 32, 2, 16, true, 8, 1)         \
  X(16, 1, 32, 4, 16, true, 8, 1)        \
  X(32, 1, 32, 8, 16, true, 10, 1)       \
  X(64, 1, 64, 8, 8, true, 4, 1)         \
  X(64, 2, 128, 8, 8, true, 4, 0)        \
  SRWM_TUNING(                           \
  X(32, 2, 64, 8, 16, true, 8, 0)        \
  X(64, 3, 256, 8, 8, true, 2, 0)        \
  X(64, 4, 128, 16, 8, true, 4, 0)       \
  X(64, 5, 64, 16, 8, true, 4, 0)        \
  X(64, 6, 64, 8, 8, false, 4, 0)        \
  X(64, 7, 256, 4, 8, true, 2, 0))
