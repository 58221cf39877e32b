"""Per-lane render state: packing engine tensors into the C-ABI records.

The renderer reads two arrays per call (layout: include/gradoom_b200_layout.h):

* ``lanes``  ``(N, 32) int32`` -- pose, weapon and status-bar scalars;
* ``things`` ``(N, K, 4) int32`` viewed as 16-byte records -- one drawable actor
  each: position, sprite patch, alive / full-bright flags and blend style.

``pack_lanes`` and ``gather_things`` build them from any object that carries
the reference engine's lane tensors under the reference's attribute names
(src/gradoom/engine.py:1653-1934), which is how the environment class adapts a
state producer to the renderer.  Everything here is elementwise torch code on
the producer's device; the drawing itself happens in the CUDA library.
"""

from __future__ import annotations

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

THING_ALIVE = 1
THING_BRIGHT = 2

_SLOT_BASE_WEAPON = (0, 0, 2, 3, 5, 6, 7)
_ENEMY_WALK_FRAME_TICS = (8, 6, 4, 6, 4, 6)
_ENEMY_IDLE_FRAME_TICS = (10, 10, 8, 10, 10, 10)
_ENEMY_ATTACK_RECOVERY = (16, 20, 4, 4, 8, 8)
_TELEPORT_FOG_TOTAL_TICS = 72
_BULLET_PUFF_FRAME_TICS = 4


def _f32_bits(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous().view(torch.int32)


def _public_or_retained(public: torch.Tensor, retained: torch.Tensor) -> torch.Tensor:
    """Fixed-point coordinate the renderer uses: the retained 16.16 value unless
    the public float was changed behind it (src/gradoom/engine.py:2122-2133)."""

    visible = retained.to(torch.float32) / FIXED_UNIT
    return torch.where(public != visible, torch.round(public * FIXED_UNIT).to(torch.int64), retained)


def view_angle_bam(angle: torch.Tensor, angle_bam: torch.Tensor) -> torch.Tensor:
    """Unsigned view BAM, honouring an overridden public angle
    (src/gradoom/engine.py:10648-10658)."""

    visible = angle_bam.to(torch.float32) * BAM_TO_RADIANS
    public = torch.bitwise_and(
        torch.round(torch.remainder(angle, 2.0 * math.pi) / BAM_TO_RADIANS).to(torch.int64),
        0xFFFFFFFF,
    )
    return torch.where(angle != visible, public, angle_bam)


def active_weapon(selected_weapon: torch.Tensor, variant: torch.Tensor) -> torch.Tensor:
    """Internal weapon id 0..7 from the selected slot (src/gradoom/engine.py:4673-4676)."""

    base = torch.as_tensor(_SLOT_BASE_WEAPON, device=selected_weapon.device, dtype=torch.int64)
    alternate = (selected_weapon == 1) | (selected_weapon == 3)
    return base[selected_weapon] + (alternate & variant).to(torch.int64)


def _u32_as_i32(t: torch.Tensor) -> torch.Tensor:
    t = t.to(torch.int64) & 0xFFFFFFFF
    return torch.where(t >= (1 << 31), t - (1 << 32), t).to(torch.int32)


FLAG_SCREEN_FLASHES = 4


def pack_lanes(src, thing_counts: torch.Tensor | None = None) -> torch.Tensor:
    """Build the ``(N, 32) int32`` lane records from engine-shaped tensors."""

    n = src.x.shape[0]
    dev = src.x.device
    out = torch.zeros((n, LANE_WORDS), dtype=torch.int32, device=dev)
    out[:, L_X] = _f32_bits(src.x)
    out[:, L_Y] = _f32_bits(src.y)
    out[:, L_ANGLE] = _f32_bits(src.angle)
    out[:, L_VIEW_Z] = _f32_bits(src.view_z)
    out[:, L_X_FIXED] = _public_or_retained(src.x, src._x_fixed).to(torch.int32)
    out[:, L_Y_FIXED] = _public_or_retained(src.y, src._y_fixed).to(torch.int32)
    out[:, L_ANGLE_BAM] = _u32_as_i32(view_angle_bam(src.angle, src._angle_bam))
    out[:, L_PITCH_BAM] = src._pitch_bam.to(torch.int32)
    flags = src.player_dead.to(torch.int32) | (src.mugshot_ouch.to(torch.int32) << 1)
    if getattr(src, "render_screen_flashes", False):
        # damage / bonus screen blends (src/gradoom/engine.py:15385-15397)
        flags = (flags | FLAG_SCREEN_FLASHES | (src.damage_count.to(torch.int32).clamp(0, 113) << 8)
                 | (src.bonus_count.to(torch.int32).clamp(0, 255) << 16))
    out[:, L_FLAGS] = flags
    out[:, L_EPISODE_TIME] = src.episode_time.to(torch.int32)
    out[:, L_BOB_FIXED] = src._player_bob_fixed.to(torch.int32)
    if thing_counts is not None:
        out[:, L_THINGS] = thing_counts.to(torch.int32)
    out[:, L_WEAPON] = active_weapon(src.selected_weapon, src.selected_weapon_variant).to(torch.int32)
    out[:, L_WPN_COOLDOWN] = src.weapon_state_cooldown.to(torch.int32)
    out[:, L_WPN_FIRE_COUNT] = src.weapon_fire_count.to(torch.int32)
    out[:, L_WPN_READY_TICS] = src.weapon_ready_tics.to(torch.int32)
    out[:, L_WPN_RAISE] = src.weapon_raise_cooldown.to(torch.int32)
    out[:, L_WPN_LOWER] = src.weapon_lower_cooldown.to(torch.int32)
    out[:, L_WPN_PENDING] = src.pending_weapon.to(torch.int32)
    out[:, L_HEALTH] = _f32_bits(src.health)
    out[:, L_ARMOR] = _f32_bits(src.armor)
    out[:, L_READY_AMMO] = _f32_bits(src.hud_ready_ammo)
    out[:, L_AMMO0:L_AMMO3 + 1] = _f32_bits(src.hud_ammo_counts)
    owned = (src.weapons != 0).to(torch.int32)
    shifts = torch.arange(owned.shape[1], device=dev, dtype=torch.int32)
    out[:, L_WEAPONS_OWNED] = (owned << shifts[None, :]).sum(dim=1).to(torch.int32)
    out[:, L_FACE_INDEX] = src.mugshot_face_index.to(torch.int32)
    out[:, L_PAIN_DIRECTION] = src.mugshot_pain_direction.to(torch.int32)
    out[:, L_PAIN_TICS] = src.mugshot_pain_tics.to(torch.int32)
    out[:, L_GRIN_TICS] = src.mugshot_grin_tics.to(torch.int32)
    out[:, L_ATTACK_HELD] = src.attack_held_tics.to(torch.int32)
    return out


def sprite_rotation(viewer_angle: torch.Tensor, actor_angle: torch.Tensor) -> torch.Tensor:
    """Zero-based clockwise Doom sprite rotation (src/gradoom/engine.py:13994-14009)."""

    relative = torch.remainder(viewer_angle - actor_angle + math.pi / 8, 2 * math.pi)
    return torch.remainder(torch.floor(relative / (math.pi / 4)).to(torch.int64), 8)


def _frame_from_ends(elapsed: torch.Tensor, ends: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    frame = torch.sum(elapsed[..., None] >= ends, dim=-1)
    return torch.minimum(frame, counts - 1)


class SpriteTables:
    """Device copies of the sprite id tables a Scene carries."""

    def __init__(self, scene, device):
        def t(a):
            return torch.as_tensor(np.ascontiguousarray(a), device=device, dtype=torch.int64)

        self.walk = t(scene.enemy_walk_ids)
        self.attack = t(scene.enemy_attack_ids)
        self.pain = t(scene.enemy_pain_ids)
        self.death = t(scene.enemy_death_ids)
        self.death_counts = t(scene.enemy_death_counts)
        self.death_ends = torch.cumsum(t(scene.enemy_death_durations), dim=1)
        self.xdeath = t(scene.enemy_xdeath_ids)
        self.xdeath_counts = t(scene.enemy_xdeath_counts)
        self.xdeath_ends = torch.cumsum(t(scene.enemy_xdeath_durations), dim=1)
        self.flight = t(scene.proj_flight_ids)
        self.explosion = t(scene.proj_explosion_ids)
        self.explosion_counts = t(scene.proj_explosion_counts)
        self.explosion_ends = torch.cumsum(t(scene.proj_explosion_durations), dim=1)
        self.explosion_total = t(scene.proj_explosion_durations).sum(dim=1)
        self.fog = t(scene.fog_ids)
        self.puff = t(scene.puff_ids)
        self.static = t(scene.static_ids)
        self.starts = torch.as_tensor(scene.player_starts, device=device, dtype=torch.float32)
        self.walk_tics = t(_ENEMY_WALK_FRAME_TICS)
        self.idle_tics = t(_ENEMY_IDLE_FRAME_TICS)
        self.recovery = t(_ENEMY_ATTACK_RECOVERY)


def enemy_sprite_ids(src, tab: SpriteTables) -> torch.Tensor:
    """Walk / attack / pain sprite of every enemy slot
    (src/gradoom/engine.py:14011-14077)."""

    etype = src.enemy_type.clamp(0, 5)
    viewer = torch.atan2(src.y[:, None] - src.enemy_y, src.x[:, None] - src.enemy_x)
    rot = sprite_rotation(viewer, src.enemy_angle)
    tics = src.enemy_animation_tics
    walk = torch.remainder(tics // tab.walk_tics[etype], 4).to(torch.int64)
    idle = torch.remainder(tics // tab.idle_tics[etype], 2).to(torch.int64)
    idle = torch.where(etype == 2, torch.zeros_like(idle), idle)
    walk = torch.where(src.enemy_target_slot < -1, idle, walk)
    phase, cooldown = src.enemy_attack_phase, src.enemy_cooldown
    recovering = (cooldown > (tab.recovery[etype] // 2)).to(torch.int64)
    zero = torch.zeros_like(etype)
    attack = torch.where((etype == 0) | (etype == 1), torch.where(phase == 2, recovering, zero), zero)
    heavy = (etype == 4) | (etype == 5)
    attack = torch.where(heavy & (phase == 1), (cooldown <= 8).to(torch.int64), attack)
    attack = torch.where(heavy & (phase == 2), torch.full_like(attack, 2), attack)
    attack = torch.where((etype == 3) & ((phase == 4) | (phase == 2)), torch.ones_like(attack), attack)
    attack = torch.where((etype == 3) & (phase == 3), torch.full_like(attack, 2), attack)
    animated = torch.where(phase > 0, tab.attack[etype, attack, rot], tab.walk[etype, walk, rot])
    return torch.where(src.enemy_pain_tics > 0, tab.pain[etype, rot], animated)


def gather_things(src, tab: SpriteTables, max_things: int | None = None):
    """Collect every drawable actor of every lane, in the reference's order.

    Returns ``(things (N,K,4) int32, counts (N,) int32)``.  Columns of inactive
    slots across all lanes are dropped like the reference does
    (src/gradoom/engine.py:14328-14682); per lane the record count is K and dead
    records simply carry a cleared alive flag.
    """

    dev = src.x.device
    n = src.x.shape[0]
    xs, ys, zs, alive, sprite, bright, style = [], [], [], [], [], [], []

    def emit(x, y, z, a, s, b, st, used):
        slots = torch.nonzero(torch.any(used, dim=0)).flatten()
        if slots.numel() == 0:
            return
        xs.append(x[:, slots]); ys.append(y[:, slots]); zs.append(z[:, slots])
        alive.append(a[:, slots]); sprite.append(s[:, slots].to(torch.int64))
        bright.append(b[:, slots])
        style.append(st[:, slots].to(torch.int64))

    # living enemies -------------------------------------------------------
    etype = src.enemy_type.clamp(0, 5)
    recovery = tab.recovery[etype]
    muzzle = ((etype == 1) & (src.enemy_attack_phase == 2) & (src.enemy_cooldown > (recovery // 2))) | (
        (etype == 3) & ((src.enemy_attack_phase == 2) | (src.enemy_attack_phase == 3)))
    eslots = torch.nonzero(torch.any(src.enemy_alive, dim=0)).flatten()
    esprite = enemy_sprite_ids(src, tab)
    xs.append(src.enemy_x[:, eslots]); ys.append(src.enemy_y[:, eslots]); zs.append(src.enemy_z[:, eslots])
    alive.append(src.enemy_alive[:, eslots]); sprite.append(esprite[:, eslots])
    bright.append(muzzle[:, eslots]); style.append(torch.full_like(esprite[:, eslots], -1))

    # voodoo dolls at the unused player starts ----------------------------------
    dolls = tab.starts[:-1]
    if len(dolls):
        dx = dolls[None, :, 0].expand(n, -1)
        dy = dolls[None, :, 1].expand(n, -1)
        dang = torch.deg2rad(dolls[None, :, 2]).expand(n, -1)
        viewer = torch.atan2(src.y[:, None] - dy, src.x[:, None] - dx)
        dspr = tab.walk[2, 0, sprite_rotation(viewer, dang)]
        xs.append(dx); ys.append(dy)
        zs.append(src._player_start_z[:-1][None, :].expand(n, -1))
        alive.append((~src.player_dead)[:, None].expand(-1, len(dolls)))
        sprite.append(dspr)
        bright.append(torch.zeros_like(dspr, dtype=torch.bool))
        style.append(torch.full_like(dspr, -1))

    # corpses ------------------------------------------------------------------
    dtype_ = src.enemy_death_type.clamp(0, 5)
    elapsed = src.enemy_death_elapsed.to(torch.int64)
    dframe = _frame_from_ends(elapsed, tab.death_ends[dtype_], tab.death_counts[dtype_])
    xframe = _frame_from_ends(elapsed, tab.xdeath_ends[dtype_], tab.xdeath_counts[dtype_])
    dspr = torch.where(src.enemy_death_extreme, tab.xdeath[dtype_, xframe], tab.death[dtype_, dframe])
    dying = src.enemy_death_tics > 0
    no = torch.zeros_like(dying)
    emit(src.enemy_x, src.enemy_y, src.enemy_z, dying, dspr, no, torch.full_like(dspr, -1), dying)

    # player projectiles in flight ---------------------------------------------
    ptype = src.projectile_type.clamp(0, 1)
    pang = torch.atan2(src.projectile_velocity_y, src.projectile_velocity_x)
    pview = torch.atan2(src.y[:, None] - src.projectile_y, src.x[:, None] - src.projectile_x)
    prot = sprite_rotation(pview, pang)
    pframe = torch.where(ptype == 1, torch.remainder(src.projectile_age // 6, 2).to(torch.int64),
                         torch.zeros_like(ptype))
    pspr = tab.flight[ptype, pframe, prot]
    palive = src.projectile_alive
    emit(src.projectile_x, src.projectile_y, src.projectile_z, palive, pspr, palive,
         torch.where(ptype == 1, torch.zeros_like(ptype), torch.full_like(ptype, -1)), palive)

    # enemy projectiles in flight ------------------------------------------------
    eang = torch.atan2(src.enemy_projectile_velocity_y, src.enemy_projectile_velocity_x)
    eview = torch.atan2(src.y[:, None] - src.enemy_projectile_y, src.x[:, None] - src.enemy_projectile_x)
    erot = sprite_rotation(eview, eang)
    eframe = torch.remainder(src.enemy_projectile_age // 4, 2).to(torch.int64)
    espr = tab.flight[2, eframe, erot]
    ealive = src.enemy_projectile_alive
    emit(src.enemy_projectile_x, src.enemy_projectile_y, src.enemy_projectile_z, ealive, espr, ealive,
         torch.ones_like(eframe), ealive)

    # impacts -----------------------------------------------------------------------
    def explosion(kind, remaining):
        safe = kind.clamp(0, 2)
        el = tab.explosion_total[safe] - remaining.to(torch.int64)
        frame = _frame_from_ends(el, tab.explosion_ends[safe], tab.explosion_counts[safe])
        return tab.explosion[safe, frame]

    pi_alive = src.projectile_impact_tics > 0
    pi_type = src.projectile_impact_type
    emit(src.projectile_x, src.projectile_y, src.projectile_z, pi_alive,
         explosion(pi_type, src.projectile_impact_tics), pi_alive,
         torch.where(pi_type == 1, torch.zeros_like(pi_type), torch.full_like(pi_type, -1)), pi_alive)
    ei_alive = src.enemy_projectile_impact_tics > 0
    ei_type = torch.full_like(src.enemy_projectile_age, 2, dtype=torch.int64)
    emit(src.enemy_projectile_x, src.enemy_projectile_y, src.enemy_projectile_z, ei_alive,
         explosion(ei_type, src.enemy_projectile_impact_tics), ei_alive, torch.ones_like(ei_type), ei_alive)

    # teleport fog ----------------------------------------------------------------------
    fog_alive = src.teleport_fog_tics > 0
    fog_frame = torch.clamp((_TELEPORT_FOG_TOTAL_TICS - src.teleport_fog_tics.to(torch.int64)) // 6, max=11)
    fog_spr = tab.fog[fog_frame]
    emit(src.teleport_fog_x, src.teleport_fog_y, src.teleport_fog_z, fog_alive, fog_spr, fog_alive,
         torch.ones_like(fog_spr), fog_alive)

    # bullet puffs ----------------------------------------------------------------------
    ptics = src.hitscan_puff_tics
    pf = torch.where(ptics > 3 * _BULLET_PUFF_FRAME_TICS, 0,
                     torch.where(ptics > 2 * _BULLET_PUFF_FRAME_TICS, 1,
                                 torch.where(ptics > _BULLET_PUFF_FRAME_TICS, 2, 3))).to(torch.int64)
    puff_spr = tab.puff[pf]
    emit(src.hitscan_puff_x, src.hitscan_puff_y, src.hitscan_puff_z, ptics > 0, puff_spr, pf == 0,
         torch.full_like(puff_spr, -2), ptics > 0)

    # map items are not generated by the synthetic scenes; dropped items ------------------
    drop_visible = (src.drop_type >= 0) & src.drop_spawned
    drop_spr = tab.static[12].expand_as(src.drop_type)
    drop_spr = torch.where(src.drop_type == 2007, tab.static[6], drop_spr)
    drop_spr = torch.where(src.drop_type == 2002, tab.static[14], drop_spr)
    emit(src.drop_x, src.drop_y, src.drop_z, drop_visible, drop_spr, torch.zeros_like(drop_visible),
         torch.full_like(drop_spr, -1), drop_visible)

    ax = torch.cat(xs, dim=1).to(torch.float32)
    ay = torch.cat(ys, dim=1).to(torch.float32)
    az = torch.cat(zs, dim=1).to(torch.float32)
    aalive = torch.cat(alive, dim=1)
    aspr = torch.cat(sprite, dim=1)
    abright = torch.cat(bright, dim=1)
    astyle = torch.cat(style, dim=1)
    k = ax.shape[1]
    if max_things is not None:
        if k > max_things:
            raise ValueError(f"{k} drawable actors exceed the configured maximum of {max_things}")
    things = pack_things(ax, ay, az, aspr, aalive, abright, astyle, pad_to=max_things)
    counts = torch.full((n,), k, dtype=torch.int32, device=dev)
    return things, counts


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
