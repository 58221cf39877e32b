/*
 * Device-side view of the scene blob and small exact-arithmetic helpers shared
 * by the render kernels.  Everything is integer 16.16 / 20.12 fixed point on
 * 64-bit integers or separately rounded float32 (the library is compiled with
 * -fmad=false), because the results must equal the reference's
 * (src/gradoom/engine.py:10534-15457) bit for bit.
 */
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/gradoom_b200_layout.h"

typedef long long i64;

#define GD_FU 65536LL
#define GD_SW GD_SCREEN_W
#define GD_VH GD_VIEW_H
#define GD_ANG90 (1LL << 30)
#define GD_FOCAL_X (160LL * GD_FU)
#define GD_Y_ASPECT ((320LL * GD_FU * 240LL) / (200LL * 320LL))
#define GD_FOCAL_Y (160LL * GD_Y_ASPECT)
#define GD_FLOOR_VIS ((160LL * GD_FU * (8LL * GD_FU)) / GD_FOCAL_Y)
#define GD_WALL_VIS (((GD_FOCAL_Y * (320LL * 600LL) / (320LL * 240LL * 3LL)) * (8LL * GD_FU)) >> 16)
#define GD_SPRITE_MIN_DEPTH (2048LL * 4LL)
#define GD_U32MASK 0xFFFFFFFFLL

/* status bits written to the device status word */
#define GD_STATUS_EVENT_OVERFLOW 1   /* a column produced more clip events than the scratch holds */
#define GD_STATUS_THINGS_OVERFLOW 2  /* a lane lists more things than the configured maximum */
#define GD_STATUS_BAD_SECTOR 4       /* checked build: a sector index outside the scene */
#define GD_STATUS_BAD_INDEX 8        /* checked build: a wall, texture, sprite or patch index outside its table */
#define GD_STATUS_BAD_STATE 16       /* checked build: a lane or thing record with a value outside its range */

struct GdScene {
  int W, S, T, texH, texW, P, sprH, sprW, Q, wpnH, wpnW, wpnTics, nStarts, B, nbDirect, wpnAvailable, hudPatches;
  const float *walls;
  const int32_t *wsec;
  const float *wlen;
  const int32_t *sideTex;
  const float *sideOff;
  const int32_t *wvtx, *vtxOff, *vtxWalls;
  const int32_t *nbDirectTab, *nbOff, *nbIdx, *nbFlags;
  const int32_t *sbStartOff, *sbStartIdx, *sbEndOff, *sbEndIdx;
  const float *secF;
  const int32_t *secI;
  const int32_t *secOff, *secWalls, *edgeOff, *edgeWalls, *blocking;
  const int32_t *texInfo;
  const uint8_t *texAtlas, *texAtlasCol, *playpal, *colormap;
  const int32_t *sprInfo;
  const uint8_t *sprAtlas, *sprPost;
  const uint8_t *addLut, *transLut;
  const int32_t *wpnInfo;
  const uint8_t *wpnAtlas, *wpnOpaque;
  const int32_t *wpnFrameIds, *wpnFlashIds, *wpnFlashLights;
  const int32_t *hudInfo;
  const uint8_t *hudAtlas, *hudOpaque;
  const int32_t *fineSine, *fineTan;
  const float *rayOffsets, *rayCosCorr;
  const float *secBBox;
  const int32_t *maskedWalls;   /* M two-sided walls that carry a middle texture */
  const float *damageAlpha;     /* 114: damage count -> red flash alpha */
  /* sectors grouped by floor / ceiling height, nearest plane first */
  const float *groupH[2];       /* [0] ceilings ascending, [1] floors descending */
  const int32_t *groupOff[2], *groupSec[2];
  int groups[2];
  int M;
  /* projection fragments of the lines a node builder split: total count, CSR per line, 16.16 endpoints */
  int F;
  const int32_t *fragOff, *fragFixed;
  /* bullet-chip decals: variants (0 = none), atlas slice height / width */
  int decals, decalH, decalW;
  const int32_t *decalInfo, *wallFine;
  const uint8_t *decalAtlas, *decalOpacity, *decalBlack;
};

/*
 * Checked build (-DGD_CHECKED, libgradoom_b200_checked.so): every index taken from
 * the scene blob, a lane record or a thing record is range-tested where it is about
 * to address memory; an index out of range is replaced by 0 (the access it would
 * have made is skipped) and a bit is set in the caller's status word.  Nothing
 * traps.  The regular build compiles the tests away.
 */
#ifdef GD_CHECKED
__device__ int *gdCheckedStatus;     /* the status word of the launch in flight (one launch at a time) */
__device__ __forceinline__ int gd_checked(int i, int n, int bit) {
  if ((unsigned)i < (unsigned)n) return i;
  atomicOr(gdCheckedStatus, bit);
  return 0;
}
#define GD_CHECK_INDEX(i, n) gd_checked((int)(i), (int)(n), GD_STATUS_BAD_INDEX)
#define GD_CHECK_SECTOR(i, n) gd_checked((int)(i), (int)(n), GD_STATUS_BAD_SECTOR)
#define GD_FLAG_STATE(bad) do { if (bad) atomicOr(gdCheckedStatus, GD_STATUS_BAD_STATE); } while (0)
#else
#define GD_CHECK_INDEX(i, n) (i)
#define GD_CHECK_SECTOR(i, n) (i)
#define GD_FLAG_STATE(bad) do { } while (0)
#endif

/* sector on one side of a wall: entry `i` of the wall-sector table, -1 = none */
__device__ __forceinline__ int gd_wsec(const GdScene &sc, int i) {
  const int s = sc.wsec[i];
#ifdef GD_CHECKED
  if (s < -1 || s >= sc.S) { atomicOr(gdCheckedStatus, GD_STATUS_BAD_SECTOR); return -1; }
#endif
  return s;
}

/* The CTA's dynamic shared memory. */
extern __shared__ __align__(16) uint8_t gd_smem[];

/* Shared-memory accesses of the pixel loops by 32-bit shared-space address: the pointers of the shared-memory
 * map are generic (they are read from a structure), so the compiler would otherwise carry 64-bit addresses
 * and issue generic loads and stores.  The loads are for tables nothing writes while a lane is drawn. */
__device__ __forceinline__ unsigned gd_shared_addr(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
/* The same pointer, re-derived from the shared array itself: the compiler then knows its address space and
 * addresses everything reached through it with 32 bits and shared-space instructions. */
template <class T>
__device__ __forceinline__ T *gd_as_shared(T *p) {
  return (T *)(gd_smem + (int)(gd_shared_addr(p) - gd_shared_addr(gd_smem)));   /* static shared variables lie below */
}
__device__ __forceinline__ unsigned gd_lds8(unsigned addr) {
  unsigned v;
  asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned gd_lds32(unsigned addr) {
  unsigned v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void gd_sts8(unsigned addr, unsigned v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ i64 gd_min(i64 a, i64 b) { return a < b ? a : b; }
__device__ __forceinline__ i64 gd_max(i64 a, i64 b) { return a > b ? a : b; }
__device__ __forceinline__ i64 gd_clamp(i64 v, i64 lo, i64 hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ i64 gd_wmul(i64 a, i64 b) { return (i64)((unsigned long long)a * (unsigned long long)b); }
__device__ __forceinline__ i64 gd_shl(i64 a, int k) { return (i64)((unsigned long long)a << k); }
/* float32 -> int64, round half to even */
__device__ __forceinline__ i64 gd_rint(float v) { return (i64)rintf(v); }
__device__ __forceinline__ i64 gd_pymod(i64 a, i64 m) {
  i64 r = a % m;
  return (r != 0 && ((r < 0) != (m < 0))) ? r + m : r;
}
/* the same for a texture width: a power of two needs no division */
__device__ __forceinline__ int gd_pymod_width(i64 a, int w) {
  if (w > 0 && (w & (w - 1)) == 0) return (int)(a & (i64)(w - 1));
  return (int)gd_pymod(a, w);
}

/*
 * Truncating signed 64-bit division.  The generic 64-bit divide is a long
 * software routine on the GPU; nearly every quotient on this path has operands
 * below 2^52, where a double-precision divide is within one of the exact
 * quotient and an integer remainder check makes it exact.
 */
__device__ __noinline__ i64 gd_div_generic(i64 a, i64 b) { return a / b; }

__device__ __noinline__ i64 gd_div(i64 a, i64 b) {
  unsigned long long ua = a < 0 ? 0ull - (unsigned long long)a : (unsigned long long)a;
  unsigned long long ub = b < 0 ? 0ull - (unsigned long long)b : (unsigned long long)b;
  if (((ua | ub) >> 52) != 0 || ub == 0) return gd_div_generic(a, b);
  i64 q = (i64)__ddiv_rn((double)ua, (double)ub);
  i64 r = (i64)ua - q * (i64)ub;
  if (r < 0) q -= 1;
  else if (r >= (i64)ub) q += 1;
  return ((a ^ b) < 0) ? -q : q;
}

struct GdView {
  float x, y, angle, viewZ;
  i64 vx, vy, pitchBam;
  i64 vsin, vcos;
  float fcos, fsin;
  i64 center;
  i64 upperClip, lowerClip;  /* view frustum top / bottom slopes used by the row projection */
  int flashLight;
};

/* Per-wall record kept in shared memory for the lane being drawn. */
struct __align__(8) GdWall {
  i64 visL[2], visStep[2], visSl[2];  /* wallscan light per side */
  i64 sl, sr;                         /* projected half-open span (unbounded when rejected) */
  i64 dl, dr;                         /* clipped endpoint depths, 20.12 */
  int tx[2], ty[2];                   /* view coordinates in stored endpoint order */
  short isl, isr;                     /* span owned by the column-ray test */
  unsigned char hasColumns, frontF, oneSided, pad;
};

/* One clip event of a column: what a drawn seg contributes to sprite clipping
 * and to visplane ownership. Rows are 0..208 and fit a byte. */
struct __align__(4) GdEvent {
  float dist;
  short wall;      /* wall whose depth clips sprites */
  short sector;    /* sector owning the planes marked by this event, -1 none */
  unsigned char t0a, t0b, t1a, t1b;  /* rows drawn by this event: two tier ranges */
  unsigned char silTop, silBot;      /* silhouettes: rows < silTop and rows >= silBot */
  unsigned char ceilA, ceilB, floorA, floorB;  /* plane marks */
  unsigned char pad0, pad1;
};

#define GD_MAX_EVENTS 48

/* Row projection of one (wall, plane height) pair: everything of the OWallMost
 * replay that does not depend on the screen column. */
struct __align__(8) GdRowProj {
  i64 pl, pstep, cl;     /* clipped-edge projection: center + pl + (x - cl) * pstep */
  i64 opl, ostep;        /* whole-wall projection for columns outside the seg's span */
  short topA, topB;      /* columns forced to row 0 (above the view frustum) */
  short botA, botB;      /* columns forced to the bottom row */
  short collapsedX;      /* the one column exempt from both, or -1 */
  unsigned char entAbove, entBelow;
  short pad;
};
