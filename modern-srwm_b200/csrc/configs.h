// Compiled kernel configurations: X(E, variant, P, R, T, PK, MINB)
//   E      head dimension            P     threads per sequence (= CTA size)
//   R      state rows per thread     T     time steps staged per chunk
//   PK     packed fma.rn.f32x2 (1) or scalar fma (0)
//   MINB   CTAs per SM the register allocation is bounded for (__launch_bounds__)
// Variant 0 is what the library uses by default; the others exist so that alternative
// tilings can be timed against each other through the same ABI.
#pragma once

#define SRWM_FWD_CONFIGS(X)      \
  X(8, 0, 32, 2, 16, true, 8)    \
  X(16, 0, 32, 4, 16, true, 8)   \
  X(16, 1, 32, 2, 16, true, 8)   \
  X(32, 1, 64, 8, 16, true, 6)   \
  X(32, 2, 32, 8, 16, true, 8)   \
  X(32, 3, 64, 4, 16, true, 6)   \
  X(64, 1, 128, 8, 16, true, 3)  \
  X(64, 2, 128, 16, 16, true, 3) \
  X(64, 3, 128, 8, 16, false, 3)

// Column-layout forward (96 threads, one warp per block): Y(E, variant, T, PK, MINB, DPRE, NRP)
//   DPRE  the k warp publishes q-k once per step (two-warp named barrier) instead of every
//         thread recomputing it in the second pass
//   NRP   row parts per column group (1 = whole columns per lane)
#define SRWM_FWD_COL_CONFIGS(Y)     \
  Y(64, 0, 16, true, 4, true, 1)    \
  Y(64, 4, 16, true, 4, false, 1)   \
  Y(64, 5, 16, true, 4, true, 2)    \
  Y(64, 6, 16, true, 4, true, 4)    \
  Y(64, 7, 16, false, 4, true, 2)   \
  Y(64, 8, 16, true, 3, true, 2)    \
  Y(16, 2, 16, true, 8, true, 2)    \
  Y(16, 3, 16, true, 16, true, 2)   \
  Y(32, 0, 16, true, 8, true, 2)    \
  Y(32, 4, 16, true, 8, false, 1)   \
  Y(32, 5, 16, true, 8, true, 1)    \
  Y(32, 6, 16, true, 8, true, 4)    \
  Y(32, 7, 16, true, 12, true, 4)

#define SRWM_BWD_CONFIGS(X)      \
  X(8, 0, 32, 2, 16, true, 8)    \
  X(16, 0, 32, 2, 16, true, 8)   \
  X(16, 1, 32, 4, 16, true, 8)   \
  X(32, 0, 64, 4, 16, true, 6)   \
  X(32, 1, 64, 8, 16, true, 6)   \
  X(32, 2, 32, 8, 16, true, 8)   \
  X(64, 0, 128, 8, 16, true, 2)  \
  X(64, 1, 256, 8, 16, true, 1)  \
  X(64, 2, 128, 8, 16, false, 2)

// Backward with the state detached at every step (W_y and its gradient only)
#define SRWM_BWD_DET_CONFIGS(X)  \
  X(8, 0, 32, 2, 16, true, 8)    \
  X(16, 0, 32, 4, 16, true, 8)   \
  X(32, 0, 64, 8, 16, true, 6)   \
  X(64, 0, 128, 16, 16, true, 4)

#define DELTA_FWD_CONFIGS(X)     \
  X(8, 0, 32, 2, 16, true, 8)    \
  X(16, 0, 32, 4, 16, true, 8)   \
  X(32, 0, 32, 8, 16, true, 12)  \
  X(32, 1, 64, 8, 16, true, 8)   \
  X(64, 6, 64, 16, 8, true, 8)   \
  X(64, 1, 64, 32, 8, true, 8)   \
  X(64, 2, 64, 64, 8, true, 8)   \
  X(64, 3, 128, 16, 8, true, 6)  \
  X(64, 4, 32, 16, 8, true, 10)  \
  X(64, 5, 64, 16, 8, false, 8)

// Column-layout delta forward: Y(E, variant, P, T, PK, MINB, NRP); the default at E = 64
#define DELTA_FWD_COL_CONFIGS(Y)  \
  Y(64, 0, 32, 8, true, 8, 1)     \
  Y(64, 7, 32, 8, true, 8, 2)     \
  Y(64, 8, 64, 8, true, 7, 2)     \
  Y(32, 2, 32, 16, true, 16, 1)   \
  Y(32, 3, 32, 16, true, 16, 2)

#define DELTA_BWD_CONFIGS(X)     \
  X(8, 0, 32, 2, 16, true, 8)    \
  X(16, 0, 32, 4, 16, true, 8)   \
  X(32, 0, 32, 8, 16, true, 10)  \
  X(32, 1, 64, 8, 16, true, 8)   \
  X(64, 0, 64, 8, 8, true, 4)    \
  X(64, 1, 128, 8, 8, true, 4)   \
  X(64, 2, 128, 16, 8, true, 4)  \
  X(64, 3, 64, 16, 8, true, 4)   \
  X(64, 4, 64, 8, 8, false, 4)
