/*
 * C ABI of the B200 render-to-observation library (libgradoom_b200.so).
 *
 * The library draws, for a batch of environment lanes, the reference's native
 * 320x208 palette-indexed Doom view (walls, visplanes, sprites, weapon, status
 * bar) and reduces it to the 84x84 grayscale policy observation, writing it
 * into the four-frame stack.  Every pointer below is a plain device or host
 * pointer; no framework types cross this boundary.  The caller owns all
 * memory: the library never allocates device memory and never blocks on the
 * host.  All device buffers must be 16-byte aligned.
 *
 * Input formats (scene blob, lane records, thing records):
 * gradoom_b200_layout.h.
 *
 * Return value: GD_OK or a negative GD_ERR_* for host-side validation
 * failures.  A call over n = 0 lanes returns GD_OK without looking at its
 * buffers.  Device-side anomalies set bits in the caller's `status` word
 * (GD_STATUS_*), which the caller reads when it wants to; kernels never trap.
 */
#ifndef GRADOOM_B200_H
#define GRADOOM_B200_H

#include <stddef.h>
#include <stdint.h>

#include "gradoom_b200_layout.h"

#ifdef __cplusplus
extern "C" {
#endif

enum gd_error {
  GD_OK = 0,
  GD_ERR_NULL = -1,
  GD_ERR_BLOB = -2,
  GD_ERR_UNSUPPORTED = -3,
  GD_ERR_SIZE = -4,
  GD_ERR_ALIGN = -5,
  GD_ERR_CUDA = -6,
  GD_ERR_SCRATCH = -7,
  GD_ERR_SHARED = -8,
  GD_ERR_STATIC_LIMIT = -9,
  GD_ERR_DEVICE = -10
};

/* device status bits */
#define GD_STATUS_EVENT_OVERFLOW 1
#define GD_STATUS_THINGS_OVERFLOW 2
/* set only by the checked build of the library (libgradoom_b200_checked.so, compiled with
 * -DGD_CHECKED), which range-tests every index taken from the blob and the records, skips the
 * access an index out of range would have made, and reports it here: */
#define GD_STATUS_BAD_SECTOR 4     /* a sector index outside the scene */
#define GD_STATUS_BAD_INDEX 8      /* a wall, texture, sprite or patch index outside its table */
#define GD_STATUS_BAD_STATE 16     /* a lane or thing record with a value outside its range */

typedef struct gd_renderer gd_renderer;

const char *gd_error_string(int code);

/*
 * Bind a renderer to a scene blob already resident on `device`.
 * Replaces: DeviceScenario.from_host + the renderer-related part of
 * TorchDeathmatchEngine.__init__ (src/gradoom/engine.py:722-1476, 1527-1634).
 * `blob_header_host` points at (at least) the first GD_HDR_WORDS*4 bytes of
 * the same blob in host memory.  `max_things` (<= 64) is the per-lane stride
 * of the thing array passed to the render calls.
 */
int gd_renderer_create(const void *blob_header_host, const void *blob_dev, size_t blob_bytes, int device,
                       int max_things, gd_renderer **out);
void gd_renderer_destroy(gd_renderer *r);

/*
 * Bullet-chip decals.  Replaces: _native_render_hitscan_decals
 * (src/gradoom/engine.py:13747-13991), the layer between the walls and the sprites.
 * `decals` is a device array of n x slots gd_decal records (16-byte aligned,
 * 1 <= slots <= GD_MAX_DECAL_SLOTS): lane l of every later render call reads
 * records [l * slots, (l + 1) * slots), the engine's per-lane ring
 * (hitscan_decal_serial / _wall / _along / _z / _style, engine.py:1870-1884) packed
 * as gd_decal.  The array must stay alive and hold at least as many lanes as the
 * calls draw.  NULL unbinds.  The layer draws only when the scene blob carries
 * decal bitmaps (GD_H_DECALS > 0).  The call may allocate (the renderer keeps its
 * own projection scratch, slots * 32 bytes per CTA) and must not overlap with
 * render calls of the same renderer; the render calls themselves stay allocation
 * free.  Pixels the flat fallback layer alone filled (rows no seg and no visplane
 * claimed) are never shaded by a chip.
 */
int gd_renderer_bind_decals(gd_renderer *r, const void *decals, int slots);

/* Scratch the caller must provide to every render call: clip events of the
 * lanes being drawn plus, in its last 16 bytes, the kernel's lane queue.  Zero
 * the buffer once after allocating it; every launch leaves the queue at zero.
 * Launches that share a scratch buffer must not overlap on the device. */
size_t gd_renderer_scratch_bytes(const gd_renderer *r);
/* Launch shape, for reports: persistent CTAs and dynamic shared memory per CTA. */
int gd_renderer_ctas(const gd_renderer *r);
size_t gd_renderer_shared_bytes(const gd_renderer *r);
/* The same for calls that neither draw the status bar nor return a full frame (gd_render_step and
 * gd_render_reset with mask_hud, and their ring / host variants): the frame's 32 status-bar rows stay
 * off chip and their 10 KB hold more of the scene's tables (or leave the SM a larger L1). */
size_t gd_renderer_shared_bytes_view(const gd_renderer *r);

/*
 * One agent step: render every lane and push the frame onto its stack
 * (`stack`: n x 4 x 84 x 84 u8, oldest first; slots shift down by one and the
 * new frame lands in slot 3).
 * Replaces: `frame = self.render_frame(); self._finish_observation(frame)` in
 * TorchDeathmatchEngine.step (src/gradoom/engine.py:9575-9576, 9545-9547) with
 * render_frame = render_reference_frame (15436-15451).
 * mask_hud != 0: the status bar rows are black in the observation (the
 * obs_crop=(0,32,0,0) "mask" profile); otherwise the status bar is drawn.
 */
int gd_render_step(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                   uint8_t *stack, void *scratch, size_t scratch_bytes, int *status, void *stream);

/*
 * Reset fill: lanes whose `reset_mask` byte is nonzero get their new frame in
 * all four stack slots; the others are neither drawn nor touched.
 * Replaces: the tail of TorchDeathmatchEngine.reset
 * (src/gradoom/engine.py:2443-2450).
 */
int gd_render_reset(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                    const uint8_t *reset_mask, uint8_t *stack, void *scratch, size_t scratch_bytes, int *status,
                    void *stream);

/*
 * gd_render_step / gd_render_reset on a mirrored ring instead of the reference's
 * oldest-first stack, for callers that accept a strided view: `ring` is
 * n x 8 x 84 x 84 u8, the new frame goes to slots `head` and `head + 4`
 * (head = step count mod 4, 0..3), and slots head+1 .. head+4 of every lane are
 * then its last four frames, oldest first -- the same (n,4,84,84) window the
 * reference keeps (src/gradoom/engine.py:9545-9547), with a lane stride of eight
 * slots.  No old slot is read or moved: 14 KB written per lane instead of 21 KB
 * read + 28 KB written.  The reset variant writes all eight slots of the masked
 * lanes (src/gradoom/engine.py:2443-2450), so their window is the reset frame
 * four times whatever `head` is.
 * `head` is a launch parameter and the window is a host-side slice: a CUDA
 * graph that captures ring steps bakes both in, so capture them only in groups
 * of four consecutive steps starting at head 0 (a replay then advances the ring
 * exactly once around), and derive the window from the step count after the replay.
 */
int gd_render_step_ring(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                        uint8_t *ring, int head, void *scratch, size_t scratch_bytes, int *status, void *stream);
int gd_render_reset_ring(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                         const uint8_t *reset_mask, uint8_t *ring, void *scratch, size_t scratch_bytes,
                         int *status, void *stream);

/*
 * Stateless frames, any subset of (NULL = not wanted):
 *   obs_out      n x 84 x 84 u8       render_reference_frame (engine.py:15436-15451)
 *   indexed_out  n x 240 x 320 u8     _render_native_indexed_frame (15338-15379)
 *   rgb_out      n x 240 x 320 x 3 u8 render_native_frame (15453-15457), the
 *                                     frame behind GraDoomVecEnv.render()/render_lane()
 *                                     (src/gradoom/env.py:1037-1056)
 * include_hud selects whether rows 208..239 of the indexed / RGB frame carry
 * the status bar (else zeros).
 */
int gd_render_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                     int include_hud, uint8_t *obs_out, uint8_t *indexed_out, uint8_t *rgb_out, void *scratch,
                     size_t scratch_bytes, int *status, void *stream);

/*
 * One agent step that also hands out the full frame it was reduced from:
 * gd_render_step plus the indexed and/or RGB24 frame of gd_render_frames from
 * the same drawing pass.  Replaces the pair the reference runs when a caller
 * asks for images every step: the observation render inside
 * TorchDeathmatchEngine.step (src/gradoom/engine.py:9575-9576) followed by
 * render_native_frame (15453-15457) behind GraDoomVecEnv.render()
 * (src/gradoom/env.py:1055); both draw the same state, so one pass serves both.
 */
int gd_render_step_frames(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                          int include_hud, uint8_t *stack, uint8_t *indexed_out, uint8_t *rgb_out, void *scratch,
                          size_t scratch_bytes, int *status, void *stream);

/*
 * gd_render_step for callers that keep their state in host memory: queues the
 * host->device copies of the records into the caller's staging buffers
 * (`lanes_dev`, `things_dev`), the render, and the device->host copy of the
 * newest 84x84 frame of every lane into `obs_host` (n x 84 x 84 u8).  Use
 * pinned host buffers to keep the call asynchronous: a pinned (or registered,
 * 16-byte aligned) `obs_host` is written by the kernel itself as each lane
 * finishes, so no copy remains after the drawing; a pageable one is filled by
 * chunked copies that overlap the drawing of the following chunk.  Either way
 * the result is complete once `stream` has been synchronised.  Calls on one
 * renderer share its side stream and events: do not overlap two of them on
 * different streams.  Same reference call site
 * as gd_render_step (src/gradoom/engine.py:9575-9576), plus the
 * `.to("cpu")` a host-side learner performs on the observation.
 */
int gd_render_step_host(const gd_renderer *r, const int32_t *lanes_host, const void *things_host, int n,
                        int mask_hud, int32_t *lanes_dev, void *things_dev, uint8_t *stack, uint8_t *obs_host,
                        void *scratch, size_t scratch_bytes, int *status, void *stream);

/*
 * Engine-shaped lane state -> render records, on the device.
 *
 * `gd_engine_state` is a table of device pointers to the reference engine's own
 * per-lane tensors, each under the reference's attribute name and in the
 * reference's dtype (src/gradoom/engine.py:1653-1934: torch.bool as uint8_t,
 * torch.int64 as int64_t, torch.int32 as int32_t, float32 as float), row-major
 * with leading dimension n.  gd_pack_state turns them into the lane records and
 * the thing records the render calls read, in two small launches and without any
 * host synchronisation:
 *   lanes   n x 32 i32            the fields of src/gradoom/engine.py:1658-1739 the
 *                                 renderer reads (layout: gradoom_b200_layout.h)
 *   things  n x max_things x 16 B every drawable actor in the order the reference
 *                                 concatenates them
 * Replaces: the actor gathering at the head of _native_render_sprites
 * (src/gradoom/engine.py:14328-14682) with _native_enemy_sprite_ids (14011-14077),
 * _native_enemy_death_sprite_ids (14079-14104),
 * _native_projectile_explosion_sprite_ids (14106-14122), _native_enemy_fullbright
 * (14124-14136), _doom_sprite_rotation (13994-14009) and _native_item_sprite_ids
 * (14258-14317), and the view-pose selection of _native_view_fixed /
 * _native_view_angle_bam (2122-2133, 10648-10658).
 * Like the reference, a slot of an actor class is dropped only when no lane of
 * the batch uses it; every lane therefore gets the same number K of records
 * (lanes where the slot is idle carry a record with the alive flag cleared), K is
 * written to word GD_L_THINGS of every lane record, and K > max_things sets
 * GD_STATUS_THINGS_OVERFLOW (the records beyond max_things are not written).
 * `flags_scratch` is gd_pack_state_scratch_bytes() of device memory (cleared by
 * the call itself).  Pointers of an actor class whose slot count is 0 may be NULL.
 */
typedef struct gd_engine_state {
  int32_t n;
  int32_t enemy_slots;              /* enemies, corpses, teleport fog and drops share it (64) */
  int32_t projectile_slots;         /* player projectiles and their impacts (32) */
  int32_t enemy_projectile_slots;   /* (64) */
  int32_t puff_slots;               /* bullet puffs (20) */
  int32_t items;                    /* map items of the scene blob (GD_H_ITEMS) */
  int32_t render_screen_flashes;    /* nonzero: pass damage_count / bonus_count on to the renderer */
  int32_t reserved;
  /* player: n */
  const float *x, *y, *angle, *view_z, *health, *armor, *hud_ready_ammo;
  const int64_t *x_fixed, *y_fixed, *angle_bam, *pitch_bam, *player_bob_fixed;      /* _x_fixed ... */
  const int64_t *selected_weapon, *pending_weapon, *mugshot_face_index, *mugshot_pain_direction;
  const int32_t *episode_time, *weapon_state_cooldown, *weapon_fire_count, *weapon_ready_tics,
      *weapon_raise_cooldown, *weapon_lower_cooldown, *mugshot_pain_tics, *mugshot_grin_tics, *attack_held_tics,
      *damage_count, *bonus_count;                                                   /* the last two may be NULL */
  const uint8_t *player_dead, *selected_weapon_variant, *mugshot_ouch;
  const float *hud_ammo_counts;     /* n x 4 */
  const float *weapons;             /* n x 6 */
  /* enemies: n x enemy_slots */
  const float *enemy_x, *enemy_y, *enemy_z, *enemy_angle;
  const int64_t *enemy_type, *enemy_target_slot, *enemy_death_type;
  const int32_t *enemy_animation_tics, *enemy_attack_phase, *enemy_cooldown, *enemy_pain_tics, *enemy_death_tics,
      *enemy_death_elapsed;
  const uint8_t *enemy_alive, *enemy_death_extreme;
  /* teleport fog and dropped items: n x enemy_slots */
  const float *teleport_fog_x, *teleport_fog_y, *teleport_fog_z;
  const int32_t *teleport_fog_tics;
  const float *drop_x, *drop_y, *drop_z;
  const int64_t *drop_type;
  const uint8_t *drop_spawned;
  /* player projectiles: n x projectile_slots */
  const float *projectile_x, *projectile_y, *projectile_z, *projectile_velocity_x, *projectile_velocity_y;
  const int64_t *projectile_type, *projectile_impact_type;
  const int32_t *projectile_age, *projectile_impact_tics;
  const uint8_t *projectile_alive;
  /* enemy projectiles: n x enemy_projectile_slots */
  const float *enemy_projectile_x, *enemy_projectile_y, *enemy_projectile_z, *enemy_projectile_velocity_x,
      *enemy_projectile_velocity_y;
  const int32_t *enemy_projectile_age, *enemy_projectile_impact_tics;
  const uint8_t *enemy_projectile_alive;
  /* bullet puffs: n x puff_slots */
  const float *hitscan_puff_x, *hitscan_puff_y, *hitscan_puff_z;
  const int32_t *hitscan_puff_tics;
  /* map items: n x items */
  const uint8_t *item_available;
  const int32_t *item_animation_initial_tics;
} gd_engine_state;

size_t gd_pack_state_scratch_bytes(void);
int gd_pack_state(const gd_renderer *r, const gd_engine_state *state, int32_t *lanes, void *things,
                  void *flags_scratch, size_t flags_scratch_bytes, int *status, void *stream);

/*
 * Per-tic player kinematics on the device, one warp per lane: turning with the
 * keyboard ramp, thrust, bob, the wall slide with step-up over the openings under
 * the player's box, solid actors in the way, friction, view-height easing, gravity
 * and landing.  Advances every lane by `tics` game tics under the lane's button mask
 * (bit i = button i of the reference's button list, src/gradoom/actions.py:10-31) and,
 * when `lanes` is not NULL, writes the new pose into the lane records the render
 * calls read (x, y, angle, view_z, the fixed-point pose, pitch, bob, episode time).
 * Replaces, for the player's pose: _move_player, _doom_axis_slide_move and
 * _vertical_player_tick inside the tic loop of TorchDeathmatchEngine.step
 * (src/gradoom/engine.py:4344-4575, 3207-3498, 4577-4671, 9558-9573).  Weapons,
 * attacks, monsters' thinking and pickups are not part of it.
 * players: n x GD_PLAYER_WORDS i32 (gradoom_b200_layout.h); buttons: n u32;
 * `actors` (may be NULL): the solid monsters of every lane, under the reference
 * engine's names and dtypes, which block the player like the voodoo dolls of the
 * scene do.
 */
typedef struct gd_solid_actors {
  int32_t enemy_slots;
  int32_t reserved;
  const float *enemy_x, *enemy_y, *enemy_z;
  const int64_t *enemy_type, *enemy_death_type;
  const int32_t *enemy_death_tics, *enemy_death_elapsed;
  const uint8_t *enemy_alive, *enemy_death_extreme;
} gd_solid_actors;

int gd_player_tics(const gd_renderer *r, int32_t *players, const uint32_t *buttons, const gd_solid_actors *actors,
                   int n, int tics, int episode_timeout, int32_t *lanes, int *status, void *stream);

/*
 * No counterpart in the reference.  gd_render_step for callers that may not
 * allocate device memory -- a plugin inside a host process whose GPU memory
 * pool is owned and budgeted by the embedding application, or code running
 * after the framework's allocator has been frozen -- and therefore cannot
 * provide the scratch buffer.  The scratch lives in a fixed array inside the
 * library (gd_static_scratch_bytes(), about 16 MB, held by every GPU that loads
 * the library until the process exits); the call allocates and frees nothing.
 * Limits: scenes of at most gd_static_max_walls() walls (more: GD_ERR_STATIC_LIMIT)
 * and at most 32 concurrently drawing CTAs, so it is slower than gd_render_step
 * on large batches.  The renderer's device must be current (else GD_ERR_DEVICE).
 * The first call on a device looks up the array's device address; make that
 * call outside any stream capture.  All calls share the one array: two calls
 * that overlap on the GPU (different streams) race.  Between calls nothing
 * needs clearing: the kernel re-zeroes the few words that must start at zero.
 */
size_t gd_static_scratch_bytes(void);
int gd_static_max_walls(void);
int gd_render_step_static(const gd_renderer *r, const int32_t *lanes, const void *things, int n, int mask_hud,
                          uint8_t *stack, int *status, void *stream);

/*
 * Diagnostic, no counterpart in the reference.  The few float32 transcendentals of the path
 * (sprite bearing and depth, engine.py:14684-14688; sprite rotation, 13994-14009; the flat
 * fallback's ray direction, 10966-10974) are evaluated by the device's libm, the reference's by
 * ATen's CPU kernels; they may differ in the last place.  This evaluates `function` on n device
 * floats with exactly the calls the kernels make, so that a test can count how often, on the
 * arguments the renderer forms, the two disagree.  `b` is read by GD_PROBE_ATAN2F (a = y, b = x)
 * and GD_PROBE_HYPOT (sqrtf(a*a + b*b)) only.
 */
enum gd_probe_function { GD_PROBE_ATAN2F = 0, GD_PROBE_COSF = 1, GD_PROBE_SINF = 2, GD_PROBE_HYPOT = 3 };
int gd_probe_libm(int function, const float *a, const float *b, float *out, int n, void *stream);

#ifdef __cplusplus
}
#endif
#endif
