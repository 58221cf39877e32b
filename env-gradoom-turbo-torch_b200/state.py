"""Per-lane render state: record layouts and the binding of engine-shaped tensors.

The renderer reads two arrays per call (layout: include/gradoom_b200_layout.h):

* ``lanes``  ``(N, 32) int32`` -- pose, weapon and status-bar scalars;
* ``things`` ``(N, K, 4) int32`` viewed as 16-byte records -- one drawable actor
  each: position, sprite patch, alive / full-bright flags and blend style.

``EngineState`` collects, from any object that carries the reference engine's
lane tensors under the reference's attribute names and dtypes
(src/gradoom/engine.py:1653-1934), the table of device pointers
``gd_engine_state`` that the CUDA library's ``gd_pack_state`` turns into those
records (sprite-id selection, actor order and view-pose selection of
src/gradoom/engine.py:13994-14136, 14258-14317, 14328-14682, 2122-2133,
10648-10658 happen in that kernel, not here).  ``pack_things`` assembles thing
records from per-actor arrays for synthetic states and tests.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

LANE_WORDS = 32
THING_BYTES = 16
FIXED_UNIT = 1 << 16
BAM_TO_RADIANS = 2.0 * math.pi / float(1 << 32)

# word indices (enum gd_lane_word)
(L_X, L_Y, L_ANGLE, L_VIEW_Z, L_X_FIXED, L_Y_FIXED, L_ANGLE_BAM, L_PITCH_BAM, L_FLAGS,
 L_EPISODE_TIME, L_BOB_FIXED, L_THINGS, L_WEAPON, L_WPN_COOLDOWN, L_WPN_FIRE_COUNT,
 L_WPN_READY_TICS, L_WPN_RAISE, L_WPN_LOWER, L_WPN_PENDING, L_HEALTH, L_ARMOR, L_READY_AMMO,
 L_AMMO0, L_AMMO1, L_AMMO2, L_AMMO3, L_WEAPONS_OWNED, L_FACE_INDEX, L_PAIN_DIRECTION,
 L_PAIN_TICS, L_GRIN_TICS, L_ATTACK_HELD) = range(32)

# word indices of the player kinematics record (enum gd_player_word)
PLAYER_WORDS = 24
(P_X_FIXED, P_Y_FIXED, P_MOMENTUM_X, P_MOMENTUM_Y, P_ANGLE_BAM, P_PITCH_BAM, P_BOB, P_Z, P_VIEW_Z, P_VIEW_HEIGHT,
 P_DELTA_VIEW_HEIGHT, P_VELOCITY_Z, P_FLOOR_Z, P_CEILING_Z, P_PREV_FLOOR_Z, P_REACTION_TIME, P_TURN_HELD,
 P_EPISODE_TIME, P_FLAGS, P_RESERVED) = range(20)
PLAYER_DEAD = 1
PLAYER_CHAINSAW_PULL = 2

THING_ALIVE = 1
THING_BRIGHT = 2
FLAG_SCREEN_FLASHES = 4

_F32, _I64, _I32, _U8 = torch.float32, torch.int64, torch.int32, torch.uint8

# struct gd_engine_state (include/gradoom_b200.h): (field, engine attribute, dtype, trailing shape key)
# in declaration order.  Shape keys: None = (n,), an int = (n, that many), a string = (n, that slot count).
ENGINE_STATE_COUNTS = ("n", "enemy_slots", "projectile_slots", "enemy_projectile_slots", "puff_slots", "items",
                       "render_screen_flashes", "reserved")
ENGINE_STATE_POINTERS = (
    *[(f, f, _F32, None) for f in ("x", "y", "angle", "view_z", "health", "armor", "hud_ready_ammo")],
    ("x_fixed", "_x_fixed", _I64, None), ("y_fixed", "_y_fixed", _I64, None),
    ("angle_bam", "_angle_bam", _I64, None), ("pitch_bam", "_pitch_bam", _I64, None),
    ("player_bob_fixed", "_player_bob_fixed", _I64, None),
    *[(f, f, _I64, None) for f in ("selected_weapon", "pending_weapon", "mugshot_face_index",
                                   "mugshot_pain_direction")],
    *[(f, f, _I32, None) for f in ("episode_time", "weapon_state_cooldown", "weapon_fire_count", "weapon_ready_tics",
                                   "weapon_raise_cooldown", "weapon_lower_cooldown", "mugshot_pain_tics",
                                   "mugshot_grin_tics", "attack_held_tics", "damage_count", "bonus_count")],
    *[(f, f, _U8, None) for f in ("player_dead", "selected_weapon_variant", "mugshot_ouch")],
    ("hud_ammo_counts", "hud_ammo_counts", _F32, 4), ("weapons", "weapons", _F32, 6),
    *[(f, f, _F32, "enemy_slots") for f in ("enemy_x", "enemy_y", "enemy_z", "enemy_angle")],
    *[(f, f, _I64, "enemy_slots") for f in ("enemy_type", "enemy_target_slot", "enemy_death_type")],
    *[(f, f, _I32, "enemy_slots") for f in ("enemy_animation_tics", "enemy_attack_phase", "enemy_cooldown",
                                            "enemy_pain_tics", "enemy_death_tics", "enemy_death_elapsed")],
    *[(f, f, _U8, "enemy_slots") for f in ("enemy_alive", "enemy_death_extreme")],
    *[(f, f, _F32, "enemy_slots") for f in ("teleport_fog_x", "teleport_fog_y", "teleport_fog_z")],
    ("teleport_fog_tics", "teleport_fog_tics", _I32, "enemy_slots"),
    *[(f, f, _F32, "enemy_slots") for f in ("drop_x", "drop_y", "drop_z")],
    ("drop_type", "drop_type", _I64, "enemy_slots"), ("drop_spawned", "drop_spawned", _U8, "enemy_slots"),
    *[(f, f, _F32, "projectile_slots") for f in ("projectile_x", "projectile_y", "projectile_z",
                                                 "projectile_velocity_x", "projectile_velocity_y")],
    *[(f, f, _I64, "projectile_slots") for f in ("projectile_type", "projectile_impact_type")],
    *[(f, f, _I32, "projectile_slots") for f in ("projectile_age", "projectile_impact_tics")],
    ("projectile_alive", "projectile_alive", _U8, "projectile_slots"),
    *[(f, f, _F32, "enemy_projectile_slots") for f in ("enemy_projectile_x", "enemy_projectile_y",
                                                       "enemy_projectile_z", "enemy_projectile_velocity_x",
                                                       "enemy_projectile_velocity_y")],
    *[(f, f, _I32, "enemy_projectile_slots") for f in ("enemy_projectile_age", "enemy_projectile_impact_tics")],
    ("enemy_projectile_alive", "enemy_projectile_alive", _U8, "enemy_projectile_slots"),
    *[(f, f, _F32, "puff_slots") for f in ("hitscan_puff_x", "hitscan_puff_y", "hitscan_puff_z")],
    ("hitscan_puff_tics", "hitscan_puff_tics", _I32, "puff_slots"),
    ("item_available", "item_available", _U8, "items"),
    ("item_animation_initial_tics", "item_animation_initial_tics", _I32, "items"),
)
_OPTIONAL = {"damage_count", "bonus_count"}
_SLOT_SOURCES = {"enemy_slots": "enemy_x", "projectile_slots": "projectile_x",
                 "enemy_projectile_slots": "enemy_projectile_x", "puff_slots": "hitscan_puff_x",
                 "items": "item_available"}


class EngineStateStruct(ctypes.Structure):
    """ctypes mirror of ``struct gd_engine_state``."""

    _fields_ = [(name, ctypes.c_int32) for name in ENGINE_STATE_COUNTS] + \
               [(field, ctypes.c_void_p) for field, _a, _d, _s in ENGINE_STATE_POINTERS]


def _as_dtype(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if dtype == _U8 and t.dtype == torch.bool:
        return t.contiguous().view(torch.uint8)      # same bytes, no copy
    if t.dtype != dtype:
        t = t.to(dtype)                              # a producer with other dtypes pays one cast
    return t.contiguous()


class EngineState:
    """The pointer table of one engine-shaped state object.

    The tensors are looked up once per call of ``refresh`` (their storage may be
    replaced by the producer between steps); tensors whose dtype already matches
    the reference's are passed without a copy.  ``keep`` holds whatever had to be
    cast so the pointers stay valid until the launch has been queued.
    """

    def __init__(self, src, *, render_screen_flashes: bool | None = None):
        self.src = src
        self.flashes = bool(getattr(src, "render_screen_flashes", False)) if render_screen_flashes is None \
            else bool(render_screen_flashes)
        self.struct = EngineStateStruct()
        self.keep: list[torch.Tensor] = []
        self.refresh()

    def refresh(self) -> "EngineState":
        src, st = self.src, self.struct
        self.keep = []
        n = int(src.x.shape[0])
        self.device = src.x.device
        st.n = n
        for count, attr in _SLOT_SOURCES.items():
            t = getattr(src, attr, None)
            setattr(st, count, 0 if t is None else int(t.shape[1]))
        st.render_screen_flashes = int(self.flashes)
        st.reserved = 0
        for field, attr, dtype, shape in ENGINE_STATE_POINTERS:
            t = getattr(src, attr, None)
            slots = shape if isinstance(shape, int) or shape is None else getattr(st, shape)
            if t is None or (isinstance(shape, str) and slots == 0):
                if t is None and field not in _OPTIONAL and not (isinstance(shape, str) and slots == 0):
                    raise AttributeError(f"the state producer has no tensor {attr!r}")
                setattr(st, field, None)
                continue
            want = (n,) if slots is None else (n, slots)
            if tuple(t.shape) != want:
                raise ValueError(f"{attr} has shape {tuple(t.shape)}, expected {want}")
            if t.device != self.device:
                raise TypeError(f"{attr} lives on {t.device}, the state on {self.device}")
            c = _as_dtype(t, dtype)
            self.keep.append(c)
            setattr(st, field, c.data_ptr())
        return self

    @property
    def n(self) -> int:
        return int(self.struct.n)


SOLID_ACTOR_POINTERS = (
    ("enemy_x", _F32), ("enemy_y", _F32), ("enemy_z", _F32), ("enemy_type", _I64), ("enemy_death_type", _I64),
    ("enemy_death_tics", _I32), ("enemy_death_elapsed", _I32), ("enemy_alive", _U8), ("enemy_death_extreme", _U8),
)


class SolidActorsStruct(ctypes.Structure):
    """ctypes mirror of ``struct gd_solid_actors``."""

    _fields_ = [("enemy_slots", ctypes.c_int32), ("reserved", ctypes.c_int32)] + \
               [(name, ctypes.c_void_p) for name, _d in SOLID_ACTOR_POINTERS]


class SolidActors:
    """Pointer table of the monsters that block the player (``gd_solid_actors``)."""

    def __init__(self, src):
        self.src = src
        self.struct = SolidActorsStruct()
        self.refresh()

    def refresh(self) -> "SolidActors":
        self.keep = []
        self.device = self.src.enemy_x.device
        self.struct.enemy_slots = int(self.src.enemy_x.shape[1])
        for name, dtype in SOLID_ACTOR_POINTERS:
            c = _as_dtype(getattr(self.src, name), dtype)
            self.keep.append(c)
            setattr(self.struct, name, c.data_ptr())
        return self


def player_records(src) -> torch.Tensor:
    """``(N,24) int32`` player kinematics records from an object that carries the reference
    engine's player tensors (src/gradoom/engine.py:1658-1744)."""

    n = src.x.shape[0]
    out = torch.zeros((n, PLAYER_WORDS), dtype=torch.int32, device=src.x.device)
    out[:, P_X_FIXED] = src._x_fixed.to(torch.int32)
    out[:, P_Y_FIXED] = src._y_fixed.to(torch.int32)
    out[:, P_MOMENTUM_X] = src._momentum_x_fixed.to(torch.int32)
    out[:, P_MOMENTUM_Y] = src._momentum_y_fixed.to(torch.int32)
    out[:, P_ANGLE_BAM] = _u32_as_i32(src._angle_bam)
    out[:, P_PITCH_BAM] = src._pitch_bam.to(torch.int32)
    out[:, P_BOB] = src._player_bob_fixed.to(torch.int32)
    for word, name in ((P_Z, "z"), (P_VIEW_Z, "view_z"), (P_VIEW_HEIGHT, "view_height"),
                       (P_DELTA_VIEW_HEIGHT, "delta_view_height"), (P_VELOCITY_Z, "velocity_z"),
                       (P_FLOOR_Z, "player_floor_z"), (P_CEILING_Z, "player_ceiling_z"),
                       (P_PREV_FLOOR_Z, "previous_player_floor_z")):
        out[:, word] = _f32_bits(getattr(src, name))
    out[:, P_REACTION_TIME] = src.reaction_time.to(torch.int32)
    out[:, P_TURN_HELD] = src.turn_held_tics.to(torch.int32)
    out[:, P_EPISODE_TIME] = src.episode_time.to(torch.int32)
    out[:, P_FLAGS] = src.player_dead.to(torch.int32) * PLAYER_DEAD + src.chainsaw_pull.to(torch.int32) * PLAYER_CHAINSAW_PULL
    return out


def decal_records(src, out: torch.Tensor | None = None) -> torch.Tensor:
    """``(N, slots, 4) int32`` decal rings (``gd_decal``: serial, wall | style << 16, along, z) from an
    object that carries the reference engine's ``hitscan_decal_*`` tensors
    (src/gradoom/engine.py:1870-1884).  With ``out`` the records are written in place (five
    elementwise launches, no host synchronisation), so a bound ring buffer follows the engine."""

    serial = src.hitscan_decal_serial
    if out is None:
        out = torch.empty((*serial.shape, 4), dtype=torch.int32, device=serial.device)
    out[..., 0] = serial.to(torch.int32)
    wall = src.hitscan_decal_wall.to(torch.int32) & 0xFFFF
    out[..., 1] = wall | (src.hitscan_decal_style.to(torch.int32) << 16)
    out[..., 2] = _f32_bits(src.hitscan_decal_along)
    out[..., 3] = _f32_bits(src.hitscan_decal_z)
    return out


def _f32_bits(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous().view(torch.int32)


def _u32_as_i32(t: torch.Tensor) -> torch.Tensor:
    t = t.to(torch.int64) & 0xFFFFFFFF
    return torch.where(t >= (1 << 31), t - (1 << 32), t).to(torch.int32)


def pack_things(x, y, z, sprite, alive, bright, style, pad_to: int | None = None) -> torch.Tensor:
    """Assemble ``(N,K,4) int32`` thing records from per-actor tensors."""

    n, k = x.shape
    kk = max(k, 1) if pad_to is None else max(pad_to, 1)
    out = torch.zeros((n, kk, 4), dtype=torch.int32, device=x.device)
    if k == 0:
        return out
    out[:, :k, 0] = _f32_bits(x)
    out[:, :k, 1] = _f32_bits(y)
    out[:, :k, 2] = _f32_bits(z)
    flags = alive.to(torch.int64) * THING_ALIVE + bright.to(torch.int64) * THING_BRIGHT
    word = (sprite.to(torch.int64) & 0xFFFF) | (flags << 16) | ((style.to(torch.int64) & 0xFF) << 24)
    out[:, :k, 3] = _u32_as_i32(word)
    return out
