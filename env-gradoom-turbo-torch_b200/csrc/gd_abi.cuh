/* The C ABI declared in include/gradoom_b200.h: renderer objects, argument validation, launches.
 * Part of gd_render.cu (one translation unit); not meant to be included elsewhere. */
#ifndef GD_ABI_CUH
#define GD_ABI_CUH

/* ---- C ABI (declared in include/gradoom_b200.h) --------------------------- */
#include "../../include/gradoom_b200.h"

#include <new>
#include <string.h>

#define GD_HOST_CHUNKS 4

struct gd_renderer {
  GdScene sc;
  int32_t header[GD_HDR_WORDS];
  const void *blobDev;
  int device;
  int maxThings;
  int ctas;
  size_t smemBytes;          /* dynamic shared memory and staged tables with the whole 240-row frame on chip ... */
  int stageMask;
  size_t smemBytesView;      /* ... and with the 208 view rows only (calls that draw no status bar and want no full
                                frame): the 10 KB go to more staged tables */
  int stageMaskView;
  int secWallsN, vtxWallsN, V;
  /* gd_render_step_host overlaps the device->host copy of one lane chunk with
   * the drawing of the next on this side stream */
  cudaStream_t copyStream;
  cudaEvent_t chunkDone[GD_HOST_CHUNKS], copiesDone;
  /* gd_renderer_bind_decals: the lanes' decal rings and the renderer's own scratch for them */
  const gd_decal *decals;
  int decalSlots;
  uint8_t *decalScratch;
  size_t decalScratchBytes;
  GdWall *fragScratch;       /* ctas x F records, allocated with the renderer when the scene has split lines */
};

static const void *gd_section(const uint8_t *dev, const int32_t *h, int s) { return dev + h[GD_HDR_SECTION0 + s]; }

extern "C" const char *gd_error_string(int code) {
  switch (code) {
    case GD_OK: return "ok";
    case GD_ERR_NULL: return "null pointer argument";
    case GD_ERR_BLOB: return "scene blob has a bad magic, version or size";
    case GD_ERR_UNSUPPORTED: return "scene uses a feature this render path does not draw";
    case GD_ERR_SIZE: return "size argument out of range";
    case GD_ERR_ALIGN: return "device pointer is not 16-byte aligned";
    case GD_ERR_CUDA: return "CUDA runtime call failed";
    case GD_ERR_SCRATCH: return "scratch buffer is too small";
    case GD_ERR_SHARED: return "scene needs more shared memory than one SM offers";
    case GD_ERR_STATIC_LIMIT: return "scene or device index exceeds the limits of the built-in scratch array";
    case GD_ERR_DEVICE: return "the renderer's device is not the current CUDA device";
    default: return "unknown error";
  }
}

/* The dynamic shared-memory limit belongs to the kernel on a device, not to one
 * renderer: every renderer raises it to the most the device allows beside the
 * kernel's static shared memory, so renderers of different scenes can live side
 * by side.  Returns that limit, or -1. */
typedef void (*gd_kernel_fn)(const GdParams);
/* the instantiation that draws a scene: with or without the code for split lines */
static gd_kernel_fn gd_kernel_for(const GdScene &sc) { return sc.F > 0 ? gd_render_kernel<true> : gd_render_kernel<false>; }

static int gd_raise_shared_limit(int maxOptin) {
  int limit = maxOptin;
  const gd_kernel_fn kernels[2] = {gd_render_kernel<false>, gd_render_kernel<true>};
  for (int k = 0; k < 2; ++k) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kernels[k]) != cudaSuccess) return -1;
    if (maxOptin - (int)fa.sharedSizeBytes < limit) limit = maxOptin - (int)fa.sharedSizeBytes;
  }
  for (int k = 0; k < 2; ++k)
    if (cudaFuncSetAttribute(kernels[k], cudaFuncAttributeMaxDynamicSharedMemorySize, limit) != cudaSuccess) return -1;
  return limit;
}

extern "C" int gd_renderer_create(const void *blob_header_host, const void *blob_dev, size_t blob_bytes, int device,
                                  int max_things, gd_renderer **out) {
  if (!blob_header_host || !blob_dev || !out) return GD_ERR_NULL;
  if (blob_bytes < GD_HDR_WORDS * 4) return GD_ERR_BLOB;
  if (((uintptr_t)blob_dev) & 15) return GD_ERR_ALIGN;
  if (max_things < 0 || max_things > 64) return GD_ERR_SIZE;
  const int32_t *h = (const int32_t *)blob_header_host;
  if (h[GD_H_MAGIC] != GD_MAGIC || h[GD_H_VERSION] != GD_VERSION || (size_t)h[GD_H_BYTES] != blob_bytes)
    return GD_ERR_BLOB;
  if (h[GD_H_UNSUPPORTED] != 0) return GD_ERR_UNSUPPORTED;
  if (h[GD_H_WALLS] <= 0 || h[GD_H_WALLS] >= 32768 || h[GD_H_SECTORS] <= 0 || h[GD_H_SECTORS] >= 32768)
    return GD_ERR_SIZE;
  gd_renderer *r = new (std::nothrow) gd_renderer;
  if (!r) return GD_ERR_CUDA;
  r->copyStream = nullptr;
  r->copiesDone = nullptr;
  r->decalScratch = nullptr;
  r->fragScratch = nullptr;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c) r->chunkDone[c] = nullptr;
  memcpy(r->header, h, sizeof r->header);
  r->device = device;
  r->blobDev = blob_dev;
  r->maxThings = max_things;
  const uint8_t *d = (const uint8_t *)blob_dev;
  GdScene &sc = r->sc;
  sc.W = h[GD_H_WALLS]; sc.S = h[GD_H_SECTORS]; sc.T = h[GD_H_TEXTURES];
  sc.texH = h[GD_H_TEX_H]; sc.texW = h[GD_H_TEX_W];
  sc.P = h[GD_H_SPRITES]; sc.sprH = h[GD_H_SPR_H]; sc.sprW = h[GD_H_SPR_W];
  sc.Q = h[GD_H_WPN_PATCHES]; sc.wpnH = h[GD_H_WPN_H]; sc.wpnW = h[GD_H_WPN_W]; sc.wpnTics = h[GD_H_WPN_TICS];
  sc.nStarts = h[GD_H_STARTS]; sc.B = h[GD_H_BLOCKING]; sc.nbDirect = h[GD_H_NB_DIRECT];
  sc.wpnAvailable = h[GD_H_WPN_AVAILABLE]; sc.hudPatches = h[GD_H_HUD_PATCHES];
#define SECP(type, name) (const type *)gd_section(d, h, name)
  sc.walls = SECP(float, GD_S_WALLS); sc.wsec = SECP(int32_t, GD_S_WALL_SECTORS); sc.wlen = SECP(float, GD_S_WALL_LEN);
  sc.sideTex = SECP(int32_t, GD_S_SIDE_TEX); sc.sideOff = SECP(float, GD_S_SIDE_OFF);
  sc.wvtx = SECP(int32_t, GD_S_WALL_VTX); sc.vtxOff = SECP(int32_t, GD_S_VTX_OFF); sc.vtxWalls = SECP(int32_t, GD_S_VTX_WALLS);
  sc.nbDirectTab = SECP(int32_t, GD_S_NB_DIRECT); sc.nbOff = SECP(int32_t, GD_S_NB_OFF);
  sc.nbIdx = SECP(int32_t, GD_S_NB_IDX); sc.nbFlags = SECP(int32_t, GD_S_NB_FLAGS);
  sc.sbStartOff = SECP(int32_t, GD_S_SB_START_OFF); sc.sbStartIdx = SECP(int32_t, GD_S_SB_START_IDX);
  sc.sbEndOff = SECP(int32_t, GD_S_SB_END_OFF); sc.sbEndIdx = SECP(int32_t, GD_S_SB_END_IDX);
  sc.secF = SECP(float, GD_S_SECTOR_F); sc.secI = SECP(int32_t, GD_S_SECTOR_I);
  sc.secOff = SECP(int32_t, GD_S_SEC_OFF); sc.secWalls = SECP(int32_t, GD_S_SEC_WALLS);
  sc.edgeOff = SECP(int32_t, GD_S_EDGE_OFF); sc.edgeWalls = SECP(int32_t, GD_S_EDGE_WALLS);
  sc.blocking = SECP(int32_t, GD_S_BLOCKING);
  sc.texInfo = SECP(int32_t, GD_S_TEX_INFO); sc.texAtlas = SECP(uint8_t, GD_S_TEX_ATLAS);
  sc.texAtlasCol = SECP(uint8_t, GD_S_TEX_ATLAS_COL);
  sc.playpal = SECP(uint8_t, GD_S_PLAYPAL); sc.colormap = SECP(uint8_t, GD_S_COLORMAP);
  sc.sprInfo = SECP(int32_t, GD_S_SPR_INFO); sc.sprAtlas = SECP(uint8_t, GD_S_SPR_ATLAS); sc.sprPost = SECP(uint8_t, GD_S_SPR_POST);
  sc.addLut = SECP(uint8_t, GD_S_ADD_LUT); sc.transLut = SECP(uint8_t, GD_S_TRANS_LUT);
  sc.wpnInfo = SECP(int32_t, GD_S_WPN_INFO); sc.wpnAtlas = SECP(uint8_t, GD_S_WPN_ATLAS); sc.wpnOpaque = SECP(uint8_t, GD_S_WPN_OPAQUE);
  sc.wpnFrameIds = SECP(int32_t, GD_S_WPN_FRAME_IDS); sc.wpnFlashIds = SECP(int32_t, GD_S_WPN_FLASH_IDS);
  sc.wpnFlashLights = SECP(int32_t, GD_S_WPN_FLASH_LIGHTS);
  sc.hudInfo = SECP(int32_t, GD_S_HUD_INFO); sc.hudAtlas = SECP(uint8_t, GD_S_HUD_ATLAS); sc.hudOpaque = SECP(uint8_t, GD_S_HUD_OPAQUE);
  sc.fineSine = SECP(int32_t, GD_S_FINESINE); sc.fineTan = SECP(int32_t, GD_S_FINETAN);
  sc.rayOffsets = SECP(float, GD_S_RAY_OFFSETS); sc.rayCosCorr = SECP(float, GD_S_RAY_COSCORR);
  sc.secBBox = SECP(float, GD_S_SECTOR_BBOX);
  sc.maskedWalls = SECP(int32_t, GD_S_MASKED_WALLS);
  sc.damageAlpha = SECP(float, GD_S_DAMAGE_ALPHA);
  sc.groupH[1] = SECP(float, GD_S_FLOOR_GROUP_H); sc.groupOff[1] = SECP(int32_t, GD_S_FLOOR_GROUP_OFF);
  sc.groupSec[1] = SECP(int32_t, GD_S_FLOOR_GROUP_SEC); sc.groups[1] = h[GD_H_FLOOR_GROUPS];
  sc.groupH[0] = SECP(float, GD_S_CEIL_GROUP_H); sc.groupOff[0] = SECP(int32_t, GD_S_CEIL_GROUP_OFF);
  sc.groupSec[0] = SECP(int32_t, GD_S_CEIL_GROUP_SEC); sc.groups[0] = h[GD_H_CEIL_GROUPS];
  sc.M = h[GD_H_MASKED_WALLS_N];
  sc.decals = h[GD_H_DECALS]; sc.decalH = h[GD_H_DECAL_H]; sc.decalW = h[GD_H_DECAL_W];
  sc.decalInfo = SECP(int32_t, GD_S_DECAL_INFO); sc.wallFine = SECP(int32_t, GD_S_WALL_FINE);
  sc.decalAtlas = SECP(uint8_t, GD_S_DECAL_ATLAS); sc.decalOpacity = SECP(uint8_t, GD_S_DECAL_OPACITY);
  sc.decalBlack = SECP(uint8_t, GD_S_DECAL_BLACK);
  sc.F = h[GD_H_FRAGMENTS]; sc.fragOff = SECP(int32_t, GD_S_FRAG_OFF); sc.fragFixed = SECP(int32_t, GD_S_FRAG_FIXED);
  r->decals = nullptr; r->decalSlots = 0; r->decalScratch = nullptr; r->decalScratchBytes = 0;
  r->fragScratch = nullptr;
#undef SECP
  r->smemBytes = gd_shared_bytes(sc.W, max_things, GD_SCREEN_H);
  r->smemBytesView = gd_shared_bytes(sc.W, max_things, GD_VH);
  r->secWallsN = h[GD_H_SEC_WALLS_N]; r->vtxWallsN = h[GD_H_VTX_WALLS_N]; r->V = h[GD_H_VERTICES];
  r->stageMask = r->stageMaskView = 0;
  int prev = 0;
  if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(device) != cudaSuccess) { delete r; return GD_ERR_CUDA; }
  int maxOptin = 0, sms = 0;
  cudaDeviceGetAttribute(&maxOptin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  int rc = GD_OK;
  const int limit = gd_raise_shared_limit(maxOptin);
  if (limit < 0) {
    rc = GD_ERR_CUDA;
  } else if ((size_t)limit < r->smemBytes) {
    rc = GD_ERR_SHARED;
  } else {
    /* stage as many topology tables as the SM's shared memory still holds */
    for (int bit = 1; bit <= GD_STAGE_ROWPROJ; bit <<= 1) {
      size_t extra = gd_stage_bytes(bit, sc.W, sc.S, r->V, r->secWallsN, r->vtxWallsN);
      if (r->smemBytes + extra <= (size_t)limit) { r->smemBytes += extra; r->stageMask |= bit; }
      if (r->smemBytesView + extra <= (size_t)limit) { r->smemBytesView += extra; r->stageMaskView |= bit; }
    }
    int perSm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, gd_kernel_for(sc), GD_THREADS, r->smemBytes) != cudaSuccess ||
        perSm < 1)
      rc = GD_ERR_CUDA;
    else
      r->ctas = sms * perSm;  /* one persistent CTA per resident slot */
  }
  if (rc == GD_OK && sc.F > 0) {
    void *mem = nullptr;
    if (cudaMalloc(&mem, (size_t)r->ctas * sc.F * sizeof(GdWall)) != cudaSuccess) rc = GD_ERR_CUDA;
    r->fragScratch = (GdWall *)mem;
  }
  r->copyStream = nullptr;
  r->copiesDone = nullptr;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c) r->chunkDone[c] = nullptr;
  if (rc == GD_OK) {
    bool ok = cudaStreamCreateWithFlags(&r->copyStream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&r->copiesDone, cudaEventDisableTiming) == cudaSuccess;
    for (int c = 0; ok && c < GD_HOST_CHUNKS; ++c)
      ok = cudaEventCreateWithFlags(&r->chunkDone[c], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) rc = GD_ERR_CUDA;
  }
  cudaSetDevice(prev);
  if (rc != GD_OK) { cudaGetLastError(); gd_renderer_destroy(r); return rc; }
  *out = r;
  return GD_OK;
}

extern "C" void gd_renderer_destroy(gd_renderer *r) {
  if (!r) return;
  int prev = 0;
  bool switched = cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(r->device) == cudaSuccess;
  for (int c = 0; c < GD_HOST_CHUNKS; ++c)
    if (r->chunkDone[c]) cudaEventDestroy(r->chunkDone[c]);
  if (r->copiesDone) cudaEventDestroy(r->copiesDone);
  if (r->copyStream) cudaStreamDestroy(r->copyStream);
  if (r->decalScratch) cudaFree(r->decalScratch);
  if (r->fragScratch) cudaFree(r->fragScratch);
  if (switched) cudaSetDevice(prev);
  delete r;
}

extern "C" int gd_renderer_bind_decals(gd_renderer *r, const void *decals, int slots) {
  if (!r) return GD_ERR_NULL;
  if (!decals) { r->decals = nullptr; r->decalSlots = 0; return GD_OK; }
  if (slots < 1 || slots > GD_MAX_DECAL_SLOTS) return GD_ERR_SIZE;
  if ((uintptr_t)decals & 15) return GD_ERR_ALIGN;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;
  const size_t need = (size_t)r->ctas * gd_decal_scratch_per_cta(slots);
  if (need > r->decalScratchBytes) {
    if (r->decalScratch) cudaFree(r->decalScratch);      /* waits for work that still uses it */
    r->decalScratch = nullptr; r->decalScratchBytes = 0;
    r->decals = nullptr; r->decalSlots = 0;
    void *mem = nullptr;
    if (cudaMalloc(&mem, need) != cudaSuccess) { cudaGetLastError(); return GD_ERR_CUDA; }
    r->decalScratch = (uint8_t *)mem; r->decalScratchBytes = need;
  }
  r->decals = (const gd_decal *)decals; r->decalSlots = slots;
  return GD_OK;
}

extern "C" size_t gd_renderer_scratch_bytes(const gd_renderer *r) {
  return r ? (size_t)r->ctas * gd_scratch_per_cta(r->sc.W, r->sc.S) + 16 : 0;
}

extern "C" int gd_renderer_ctas(const gd_renderer *r) { return r ? r->ctas : 0; }
extern "C" size_t gd_renderer_shared_bytes(const gd_renderer *r) { return r ? r->smemBytes : 0; }
extern "C" size_t gd_renderer_shared_bytes_view(const gd_renderer *r) { return r ? r->smemBytesView : 0; }

static int gd_launch(const gd_renderer *r, const int32_t *lanes, const gd_thing *things, int n, int flags,
                     uint8_t *stack, const uint8_t *reset_mask, uint8_t *obs_out, uint8_t *indexed_out,
                     uint8_t *rgb_out, void *scratch, size_t scratch_bytes, int *status, void *stream,
                     int ring_head = 0) {
  if (!r || !lanes || !scratch || !status) return GD_ERR_NULL;
  if (r->maxThings > 0 && !things) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (n == 0) return GD_OK;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;   /* the launch goes to the current device */
  if (scratch_bytes < gd_renderer_scratch_bytes(r)) return GD_ERR_SCRATCH;
  uintptr_t align = (uintptr_t)lanes | (uintptr_t)things | (uintptr_t)stack | (uintptr_t)obs_out |
                    (uintptr_t)indexed_out | (uintptr_t)rgb_out | (uintptr_t)scratch;
  if (align & 15) return GD_ERR_ALIGN;
  GdParams p;
  p.sc = r->sc;
  p.lanes = lanes; p.things = things; p.maxThings = r->maxThings; p.n = n; p.flags = flags;
  p.stack = stack; p.ringHead = ring_head; p.resetMask = reset_mask; p.obsOut = obs_out; p.indexedOut = indexed_out; p.rgbOut = rgb_out;
  p.scratch = (uint8_t *)scratch; p.status = status;
  p.queueOffset = (size_t)r->ctas * gd_scratch_per_cta(r->sc.W, r->sc.S);
  /* the status-bar rows of the frame stay off chip when nothing of this call shows them */
  const bool viewOnly = (flags & GD_F_MASK_HUD) && !(flags & GD_F_DRAW_HUD) && !indexed_out && !rgb_out;
  p.frameRows = viewOnly ? GD_VH : GD_SCREEN_H;
  p.stageMask = viewOnly ? r->stageMaskView : r->stageMask;
  p.secWallsN = r->secWallsN; p.vtxWallsN = r->vtxWallsN; p.V = r->V;
  p.decals = r->decals; p.decalSlots = r->decalSlots; p.decalScratch = r->decalScratch;
  p.fragScratch = r->fragScratch;
  int grid = n < r->ctas ? n : r->ctas;
  gd_kernel_for(r->sc)<<<grid, GD_THREADS, viewOnly ? r->smemBytesView : r->smemBytes, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

extern "C" int gd_render_step(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                              uint8_t *stack, void *scratch, size_t scratch_bytes, int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!stack) return GD_ERR_NULL;
  int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, nullptr, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream);
}

extern "C" int gd_render_step_ring(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                   int mask_hud, uint8_t *ring, int head, void *scratch, size_t scratch_bytes,
                                   int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!ring) return GD_ERR_NULL;
  if (head < 0 || head >= GD_STACK) return GD_ERR_SIZE;
  int flags = GD_F_STACK_RING | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, ring, nullptr, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream, head);
}

extern "C" int gd_render_reset_ring(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                    int mask_hud, const uint8_t *reset_mask, uint8_t *ring, void *scratch,
                                    size_t scratch_bytes, int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!ring || !reset_mask) return GD_ERR_NULL;
  int flags = GD_F_STACK_RING | GD_F_STACK_FILL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, ring, reset_mask, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream);
}

extern "C" int gd_render_reset(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                               const uint8_t *reset_mask, uint8_t *stack, void *scratch, size_t scratch_bytes,
                               int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!stack || !reset_mask) return GD_ERR_NULL;
  int flags = GD_F_STACK_FILL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, reset_mask, nullptr, nullptr, nullptr, scratch,
                   scratch_bytes, status, stream);
}

extern "C" int gd_render_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                                int include_hud, uint8_t *obs_out, uint8_t *indexed_out, uint8_t *rgb_out,
                                void *scratch, size_t scratch_bytes, int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!obs_out && !indexed_out && !rgb_out) return GD_ERR_NULL;
  int flags = (mask_hud ? GD_F_MASK_HUD : 0) | ((include_hud || !mask_hud) ? GD_F_DRAW_HUD : 0);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, nullptr, nullptr, obs_out, indexed_out, rgb_out,
                   scratch, scratch_bytes, status, stream);
}

extern "C" int gd_render_step_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                     int mask_hud, int include_hud, uint8_t *stack, uint8_t *indexed_out,
                                     uint8_t *rgb_out, void *scratch, size_t scratch_bytes, int *status,
                                     void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!stack || (!indexed_out && !rgb_out)) return GD_ERR_NULL;
  int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : 0) | ((include_hud || !mask_hud) ? GD_F_DRAW_HUD : 0);
  return gd_launch(r, lanes, (const gd_thing *)things, n, flags, stack, nullptr, nullptr, indexed_out, rgb_out,
                   scratch, scratch_bytes, status, stream);
}

/* Host-buffer variant of gd_render_step: copies the lane and thing records to
 * the caller's device staging buffers, renders, and copies the newest frame of
 * every lane (stack slot 3) back to `obs_host`.  Everything is queued on
 * `stream`; pinned host memory keeps the copies asynchronous. */
extern "C" int gd_render_step_host(const gd_renderer *r, const int32_t *lanes_host, const void *things_host, int n,
                                   int mask_hud, int32_t *lanes_dev, void *things_dev, uint8_t *stack,
                                   uint8_t *obs_host, void *scratch, size_t scratch_bytes, int *status,
                                   void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!r || !lanes_host || !lanes_dev || !stack || !obs_host) return GD_ERR_NULL;
  if (r->maxThings > 0 && (!things_host || !things_dev)) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (n == 0) return GD_OK;
  /* every argument is checked before the first copy is queued */
  if (!scratch || !status) return GD_ERR_NULL;
  if (scratch_bytes < gd_renderer_scratch_bytes(r)) return GD_ERR_SCRATCH;
  if (((uintptr_t)lanes_dev | (uintptr_t)things_dev | (uintptr_t)stack | (uintptr_t)scratch) & 15) return GD_ERR_ALIGN;
  {
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
    if (current != r->device) return GD_ERR_DEVICE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  size_t thingStride = (size_t)(r->maxThings > 0 ? r->maxThings : 1) * sizeof(gd_thing);
  if (cudaMemcpyAsync(lanes_dev, lanes_host, (size_t)n * GD_LANE_WORDS * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return GD_ERR_CUDA;
  if (things_host &&
      cudaMemcpyAsync(things_dev, things_host, (size_t)n * thingStride, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return GD_ERR_CUDA;
  /* Pinned (or registered) host memory is mapped into the device's address
   * space: the kernel then writes every lane's newest frame straight into it
   * while it draws the following lanes, and no copy is left to wait for. */
  {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, obs_host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr && (((uintptr_t)attr.devicePointer) & 15) == 0) {
      int flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
      return gd_launch(r, lanes_dev, (const gd_thing *)things_dev, n, flags, stack, nullptr,
                       (uint8_t *)attr.devicePointer, nullptr, nullptr, scratch, scratch_bytes, status, stream);
    }
    cudaGetLastError();
  }
  /* Pageable host memory: lanes are drawn in chunks; each chunk's newest frames travel to the host
   * on the side stream while the next chunk is drawn.  The caller's stream
   * waits for the last copy, so synchronising it covers the whole call. */
  const size_t frame = (size_t)GD_OBS * GD_OBS;
  const int chunks = n >= 512 * GD_HOST_CHUNKS ? GD_HOST_CHUNKS : 1;
  const int per = (n + chunks - 1) / chunks;
  for (int c = 0; c < chunks; ++c) {
    const int n0 = c * per, nc = (n0 + per <= n ? per : n - n0);
    if (nc <= 0) break;
    const gd_thing *th = things_dev ? (const gd_thing *)things_dev + (size_t)n0 * (r->maxThings > 0 ? r->maxThings : 1)
                                    : nullptr;
    uint8_t *st = stack + (size_t)n0 * GD_STACK * frame;
    int rc = gd_render_step(r, lanes_dev + (size_t)n0 * GD_LANE_WORDS, th, nc, mask_hud, st, scratch, scratch_bytes,
                            status, stream);
    if (rc != GD_OK) return rc;
    cudaStream_t cs = s;
    if (chunks > 1) {
      cs = r->copyStream;
      if (cudaEventRecord(r->chunkDone[c], s) != cudaSuccess || cudaStreamWaitEvent(cs, r->chunkDone[c], 0) != cudaSuccess)
        return GD_ERR_CUDA;
    }
    if (cudaMemcpy2DAsync(obs_host + (size_t)n0 * frame, frame, st + (GD_STACK - 1) * frame, GD_STACK * frame, frame,
                          (size_t)nc, cudaMemcpyDeviceToHost, cs) != cudaSuccess)
      return GD_ERR_CUDA;
  }
  if (chunks > 1) {
    if (cudaEventRecord(r->copiesDone, r->copyStream) != cudaSuccess ||
        cudaStreamWaitEvent(s, r->copiesDone, 0) != cudaSuccess)
      return GD_ERR_CUDA;
  }
  return GD_OK;
}

/* ---- allocation-free entry point ------------------------------------------
 * gd_render_step for hosts that are not allowed to allocate device memory at
 * all -- for instance a plugin loaded into an inference server or a game
 * process whose memory pool is owned and fully budgeted by its embedder, or
 * code that runs after the framework's allocator has been frozen.  Such a
 * caller cannot obtain the scratch buffer the other entry points ask for, so
 * this variant keeps the clip-event scratch in a fixed array inside the
 * library image.  Every GPU that loads the library holds GD_STATIC_SCRATCH_BYTES
 * of it until the process exits.
 */
#define GD_STATIC_MAX_CTAS 32
#define GD_STATIC_MAX_WALLS 256
/* a scene of W walls has fewer than W sectors (three walls bound a sector, a wall bounds two) */
#define GD_STATIC_PER_CTA ((GD_SCRATCH_FIXED + GD_STATIC_MAX_WALLS * 2 * GD_PLANE_ENTRY_BYTES + \
                            GD_STATIC_MAX_WALLS * 4 * sizeof(GdRowProj) + 31) & ~(size_t)15)
#define GD_STATIC_SCRATCH_BYTES (GD_STATIC_MAX_CTAS * GD_STATIC_PER_CTA + 16)
#define GD_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char gd_static_scratch[GD_STATIC_SCRATCH_BYTES];

/* device address of the array above, looked up once per device */
static unsigned char *gd_static_scratch_ptr[GD_STATIC_MAX_DEVICES];

extern "C" size_t gd_static_scratch_bytes(void) { return GD_STATIC_SCRATCH_BYTES; }
extern "C" int gd_static_max_walls(void) { return GD_STATIC_MAX_WALLS; }

extern "C" int gd_render_step_static(const gd_renderer *r, const int32_t *lanes, const void *things, int n,
                                     int mask_hud, uint8_t *stack, int *status, void *stream) {
  if (r && n == 0) return GD_OK;   /* an empty batch needs no buffers */
  if (!r || !lanes || !stack || !status) return GD_ERR_NULL;
  if (r->maxThings > 0 && !things) return GD_ERR_NULL;
  if (n < 0) return GD_ERR_SIZE;
  if (r->sc.W > GD_STATIC_MAX_WALLS || r->sc.S > GD_STATIC_MAX_WALLS) return GD_ERR_STATIC_LIMIT;
  if (r->device < 0 || r->device >= GD_STATIC_MAX_DEVICES) return GD_ERR_STATIC_LIMIT;
  if (n == 0) return GD_OK;
  uintptr_t align = (uintptr_t)lanes | (uintptr_t)things | (uintptr_t)stack;
  if (align & 15) return GD_ERR_ALIGN;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return GD_ERR_CUDA;
  if (current != r->device) return GD_ERR_DEVICE;  /* the renderer's device must be the current one */
  unsigned char *scratch = gd_static_scratch_ptr[current];
  if (!scratch) {
    /* In host code the array's name is only a handle: the kernel needs the
     * address the symbol has on this device. */
    void *address = nullptr;
    if (cudaGetSymbolAddress(&address, gd_static_scratch) != cudaSuccess || !address) {
      cudaGetLastError();
      return GD_ERR_CUDA;
    }
    scratch = (unsigned char *)address;
    gd_static_scratch_ptr[current] = scratch;
  }
  GdParams p;
  p.sc = r->sc;
  p.lanes = lanes; p.things = (const gd_thing *)things; p.maxThings = r->maxThings; p.n = n;
  p.flags = GD_F_STACK_ROLL | (mask_hud ? GD_F_MASK_HUD : GD_F_DRAW_HUD);
  p.stack = stack; p.ringHead = 0; p.resetMask = nullptr; p.obsOut = nullptr; p.indexedOut = nullptr; p.rgbOut = nullptr;
  p.scratch = scratch; p.status = status;
  /* lane queue: the last 16 bytes of the array; zero when the library is
   * loaded and left at zero by every launch */
  p.queueOffset = (size_t)GD_STATIC_MAX_CTAS * GD_STATIC_PER_CTA;
  p.frameRows = GD_SCREEN_H; p.stageMask = r->stageMask;
  p.secWallsN = r->secWallsN; p.vtxWallsN = r->vtxWallsN; p.V = r->V;
  p.decals = r->decals; p.decalSlots = r->decalSlots; p.decalScratch = r->decalScratch;
  p.fragScratch = r->fragScratch;
  int grid = n < r->ctas ? n : r->ctas;
  if (grid > GD_STATIC_MAX_CTAS) grid = GD_STATIC_MAX_CTAS;
  gd_kernel_for(r->sc)<<<grid, GD_THREADS, r->smemBytes, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

/* ---- diagnostic: the device's float32 libm on caller-given arguments -------------------- */
__global__ void gd_probe_libm_kernel(int function, const float *a, const float *b, float *out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float r;
  switch (function) {
    case GD_PROBE_ATAN2F: r = atan2f(a[i], b[i]); break;
    case GD_PROBE_COSF: r = cosf(a[i]); break;
    case GD_PROBE_SINF: r = sinf(a[i]); break;
    default: r = sqrtf(a[i] * a[i] + b[i] * b[i]); break;      /* GD_PROBE_HYPOT: the sprite distance as the kernel forms it */
  }
  out[i] = r;
}

extern "C" int gd_probe_libm(int function, const float *a, const float *b, float *out, int n, void *stream) {
  if (!a || !out || ((function == GD_PROBE_ATAN2F || function == GD_PROBE_HYPOT) && !b)) return GD_ERR_NULL;
  if (function < GD_PROBE_ATAN2F || function > GD_PROBE_HYPOT || n < 0) return GD_ERR_SIZE;
  if (n == 0) return GD_OK;
  gd_probe_libm_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(function, a, b, out, n);
  return cudaGetLastError() == cudaSuccess ? GD_OK : GD_ERR_CUDA;
}

#endif
