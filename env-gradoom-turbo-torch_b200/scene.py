"""Host-side scene description and the seeded synthetic map generator.

A :class:`Scene` is the immutable, per-device input of the renderer: map
geometry (linedef-like walls with a front sector on the right of ``v1 -> v2``
and an optional back sector), sector heights / lights / flats, the palette
indexed texture atlas, PLAYPAL, COLORMAP, sprite patches with their id tables,
psprite (weapon) patches and the status-bar patches.  Field meanings follow the
reference's ``CompiledScenario`` (src/gradoom/scenario.py:302-401) so a scene
can be converted to one and fed to the reference engine unchanged; the names
and the container are this package's own.

The generator stands in for the Doom assets, which are not redistributable and
not present: it emits grid maps of rectangular rooms joined by two-sided lines
with uniformly drawn heights, lights, textures, palette and sprite patches.
"""

from __future__ import annotations

from dataclasses import dataclass, field
import numpy as np

# Sizes of the fixed id tables the sprite stage indexes (reference defaults:
# src/gradoom/engine.py:922-1083).
ENEMY_TYPES = 6
HUD_PATCHES = 70
WEAPON_TABLE_TICS = 52


@dataclass(frozen=True)
class Scene:
    # geometry ----------------------------------------------------------
    walls: np.ndarray            # (W,4) f32  x1,y1,x2,y2
    wall_sectors: np.ndarray     # (W,2) i32  front, back (-1 = one sided)
    side_textures: np.ndarray    # (W,2,3) i32 (middle, bottom, top), -1 none
    side_offsets: np.ndarray     # (W,2,2) f32 (x, y) texel offsets
    sector_edge_mask: np.ndarray  # (S,W) bool walls bounding each sector
    sector_heights: np.ndarray   # (S,2) f32 floor, ceiling
    sector_lights: np.ndarray    # (S,) i16
    sector_floor_tex: np.ndarray  # (S,) i32
    sector_ceil_tex: np.ndarray  # (S,) i32
    player_starts: np.ndarray    # (P,3) f32 x,y,angle_deg; last row = player
    # textures ----------------------------------------------------------
    tex_atlas: np.ndarray        # (T,Hmax,Wmax) u8 palette indices
    tex_widths: np.ndarray       # (T,) i32 (powers of two)
    tex_heights: np.ndarray      # (T,) i32 (powers of two)
    playpal: np.ndarray          # (256,3) u8
    colormap: np.ndarray         # (34,256) u8
    # sprites -----------------------------------------------------------
    spr_atlas: np.ndarray        # (P,h,w) u8 palette indices
    spr_opaque: np.ndarray       # (P,h,w) bool
    spr_widths: np.ndarray       # (P,) i32
    spr_heights: np.ndarray      # (P,) i32
    spr_left: np.ndarray         # (P,) i32
    spr_top: np.ndarray          # (P,) i32
    enemy_walk_ids: np.ndarray   # (6,4,8) i32
    enemy_attack_ids: np.ndarray  # (6,4,8) i32
    enemy_pain_ids: np.ndarray   # (6,8) i32
    enemy_death_ids: np.ndarray  # (6,F) i32
    enemy_death_counts: np.ndarray     # (6,) i32
    enemy_death_durations: np.ndarray  # (6,F) i32
    enemy_xdeath_ids: np.ndarray
    enemy_xdeath_counts: np.ndarray
    enemy_xdeath_durations: np.ndarray
    proj_flight_ids: np.ndarray  # (3,2,8) i32
    proj_explosion_ids: np.ndarray  # (3,5) i32
    proj_explosion_counts: np.ndarray  # (3,) i32
    proj_explosion_durations: np.ndarray  # (3,5) i32
    fog_ids: np.ndarray          # (12,) i32
    puff_ids: np.ndarray         # (4,) i32
    static_ids: np.ndarray       # (20,) i32
    additive_luts: np.ndarray    # (2,256,256) u8 [style][dst][src]
    translucent_lut: np.ndarray  # (256,256) u8 [dst][src]
    # weapon (psprite) --------------------------------------------------
    wpn_atlas: np.ndarray        # (Q,h,w) u8
    wpn_opaque: np.ndarray       # (Q,h,w) bool
    wpn_widths: np.ndarray
    wpn_heights: np.ndarray
    wpn_left: np.ndarray
    wpn_top: np.ndarray
    wpn_frame_ids: np.ndarray    # (8,2,52) i32
    wpn_flash_ids: np.ndarray    # (8,2,52) i32 (-1 none)
    wpn_flash_lights: np.ndarray  # (8,2,52) i32
    # status bar --------------------------------------------------------
    hud_atlas: np.ndarray        # (70,32,320) u8
    hud_opaque: np.ndarray       # (70,32,320) bool
    hud_widths: np.ndarray
    hud_heights: np.ndarray
    hud_left: np.ndarray
    hud_top: np.ndarray
    meta: dict = field(default_factory=dict)

    @property
    def num_walls(self) -> int:
        return int(self.walls.shape[0])

    @property
    def num_sectors(self) -> int:
        return int(self.sector_heights.shape[0])


@dataclass(frozen=True)
class GridSpec:
    """Parameters of one seeded grid map (the synthetic-WAD stand-in)."""

    rows: int = 4
    cols: int = 4
    room: float = 256.0
    seed: int = 1
    wall_textures: int = 8
    tex_w: int = 64
    tex_h: int = 128
    flats: int = 4
    floor_max: int = 64          # floors uniform in {0, 8, ..., floor_max}
    ceil_lo: int = 128
    ceil_hi: int = 256           # ceilings uniform in {ceil_lo, +8, ..., ceil_hi}
    light_lo: int = 96
    light_hi: int = 255          # lights uniform in {96, 112, ..., <=255}
    diagonals: bool = False      # one self-referencing diagonal line per room
    mid_textures: float = 0.0    # share of two-sided lines that carry a masked middle texture
    sprite_patches: int = 96
    spr_w: int = 41
    spr_h: int = 57
    dolls: int = 1
    hud: bool = True
    weapon: bool = True
    items: int = 0               # map items (pickups) at seeded positions, cycling through the animated kinds
    decals: bool = False         # carry bullet-chip decal bitmaps and their blend tables
    splits: float = 0.0          # share of lines a node builder "split" into two or three projection fragments


# The five workloads of the benchmark definition, by name.
GRID_CONFIGS = {
    "c1": GridSpec(rows=4, cols=4, room=256.0, seed=1, wall_textures=8, flats=4,
                   floor_max=64),
    "c2": GridSpec(rows=8, cols=8, room=256.0, seed=2, wall_textures=16, flats=8,
                   floor_max=128),
    "c3": GridSpec(rows=4, cols=8, room=256.0, seed=3, wall_textures=16, flats=8,
                   floor_max=128),
    "c4": GridSpec(rows=16, cols=16, room=128.0, seed=4, wall_textures=64,
                   tex_w=128, tex_h=128, flats=8, floor_max=128, diagonals=True),
    # not a benchmark configuration: c1's shape with masked middle textures on half of the
    # two-sided lines, for the parity tests of that part of the renderer
    "c1m": GridSpec(rows=4, cols=4, room=256.0, seed=5, wall_textures=8, flats=4,
                    floor_max=64, mid_textures=0.5),
    # c1 with twelve map items, for the parity tests of the state packer
    "c1i": GridSpec(rows=4, cols=4, room=256.0, seed=1, wall_textures=8, flats=4,
                    floor_max=64, items=12),
    # c1 and a quarter-size c4 (diagonal lines) with bullet-chip decal bitmaps, for the parity tests
    # of the decal layer
    "c1d": GridSpec(rows=4, cols=4, room=256.0, seed=1, wall_textures=8, flats=4,
                    floor_max=64, decals=True),
    "c4d": GridSpec(rows=8, cols=8, room=128.0, seed=4, wall_textures=16,
                    tex_w=128, tex_h=128, flats=8, floor_max=128, diagonals=True, decals=True),
    # masked middle textures with chips on them, and the 64-sector map with chips (drawn from the poses
    # that leave most of the view to the flat fallback)
    "c1md": GridSpec(rows=4, cols=4, room=256.0, seed=5, wall_textures=8, flats=4,
                     floor_max=64, mid_textures=0.5, decals=True),
    "c2dec": GridSpec(rows=8, cols=8, room=256.0, seed=2, wall_textures=16, flats=8,
                      floor_max=128, decals=True),
    # c1 and the quarter-size diagonal map with 40 % of their lines split into projection fragments
    "c1s": GridSpec(rows=4, cols=4, room=256.0, seed=1, wall_textures=8, flats=4,
                    floor_max=64, splits=0.4),
    "c4s": GridSpec(rows=8, cols=8, room=128.0, seed=4, wall_textures=16,
                    tex_w=128, tex_h=128, flats=8, floor_max=128, diagonals=True, splits=0.4),
}


# editor type id of a map item -> index of its resting sprite in the static sprite list, counted
# from 6 as the reference does (src/gradoom/engine.py:490-508, 1084-1088)
ITEM_SPRITE_INDEX = {2011: 6, 2012: 7, 2014: 8, 2015: 9, 2018: 10, 2019: 11, 2007: 12, 2048: 13, 2049: 14,
                     2046: 15, 17: 16, 2005: 17, 2001: 18, 82: 19, 2002: 20, 2003: 21, 2004: 22}


def _sprite_patches(rng, count, w, h):
    atlas = rng.integers(1, 256, size=(count, h, w), dtype=np.uint8)
    yy, xx = np.mgrid[0:h, 0:w]
    for i in range(count):
        cx = (w - 1) / 2 + rng.uniform(-3, 3)
        cy = (h - 1) / 2 + rng.uniform(-3, 3)
        rx = w / 2 * rng.uniform(0.6, 1.0)
        ry = h / 2 * rng.uniform(0.7, 1.0)
        outside = ((xx - cx) / rx) ** 2 + ((yy - cy) / ry) ** 2 > 1.0
        holes = rng.random((h, w)) < 0.04
        atlas[i][outside | holes] = 0
    return atlas, atlas != 0


_ITEM_KINDS = (2014, 2015, 2018, 2019, 2011, 2012, 2007, 2001)   # both bonuses, both armours, four still pickups


def decal_opacity_lut() -> np.ndarray:
    """(32, 256) opacity of a chip texel under each wall shade: ZDoom's shaded-decal table for a
    `translucent 0.85` decal, alpha level 13 of 16 (definition: src/gradoom/scenario.py:260-268)."""

    texel = np.arange(256, dtype=np.int64)
    shade = np.arange(32, dtype=np.int64)[:, None]
    alpha = (32 - shade) * 256 // 32 * 13
    return np.minimum(((texel + 2) * alpha + 256) >> 14, 64).astype(np.uint8)


def _synthetic_decals(spec: GridSpec, colormap: np.ndarray) -> dict:
    """Five seeded grayscale chips, seven texels wide and five to nine tall, with holes, and the two
    blend tables: the opacity table by its definition, the darkening table from the scene's own
    colormap (opacity 0 leaves a colour alone, 64 takes it to the darkest row)."""

    rng = np.random.default_rng(spec.seed + 3000)
    heights = np.asarray((9, 7, 8, 5, 6), dtype=np.int32)
    atlas = np.zeros((5, 9, 7), dtype=np.uint8)
    for i, h in enumerate(heights):
        chip = rng.integers(1, 256, size=(h, 7)).astype(np.uint8)
        chip[rng.random((h, 7)) < 0.25] = 0
        atlas[i, :h] = chip
    rows = (np.arange(65) * 31) // 64
    return {"atlas": atlas, "heights": heights, "left": np.asarray((3, 4, 3, 2, 3), dtype=np.int32),
            "top": np.asarray((4, 3, 4, 2, 3), dtype=np.int32), "opacity_lut": decal_opacity_lut(),
            "black_lut": np.ascontiguousarray(colormap[rows]).astype(np.uint8)}


def synthetic_fragments(walls: np.ndarray, share: float, seed: int) -> dict:
    """Split a seeded share of the lines into two or three fragments at interior points, some of
    them a few fixed-point units off the line, as a node builder's rounded intersections are."""

    rng = np.random.default_rng(seed)
    fixed = np.rint(walls.astype(np.float64) * FIXED_UNIT).astype(np.int64)
    out = {}
    for w in np.flatnonzero(rng.random(len(walls)) < share):
        a, b = fixed[w, :2], fixed[w, 2:]
        cuts = (0.5,) if rng.random() < 0.6 else (float(rng.choice((0.25, 0.375))), 0.75)
        points = [a]
        for t in cuts:
            point = a + np.rint((b - a) * t).astype(np.int64)
            if rng.random() < 0.5:
                point = point + rng.integers(-3, 4, size=2)
            points.append(point)
        points.append(b)
        out[int(w)] = np.asarray([(*points[i], *points[i + 1]) for i in range(len(points) - 1)], dtype=np.int64)
    return out


def _scene_meta(spec: GridSpec, static_ids, patches) -> dict:
    meta = {"spec": spec}
    if spec.items > 0:
        # a generator of its own, so the other tables of a seed do not move
        rng = np.random.default_rng(spec.seed + 2000)
        spawns = np.zeros((spec.items, 3), dtype=np.float32)
        spawns[:, 0] = rng.uniform(24, spec.cols * spec.room - 24, size=spec.items).round()
        spawns[:, 1] = rng.uniform(24, spec.rows * spec.room - 24, size=spec.items).round()
        types = np.asarray([_ITEM_KINDS[i % len(_ITEM_KINDS)] for i in range(spec.items)], dtype=np.int32)
        meta["items"] = {"spawns": spawns, "types": types,
                         "anim_ids": rng.integers(0, patches, size=8).astype(np.int32)}
    return meta


def make_grid_scene(spec: GridSpec) -> Scene:
    rng = np.random.default_rng(spec.seed)
    R, C, room = spec.rows, spec.cols, np.float32(spec.room)
    S = R * C

    def sid(r, c):
        return r * C + c

    walls, sectors, one_sided = [], [], []

    def add(x1, y1, x2, y2, front, back):
        # ``front`` must be on the right of (x1,y1)->(x2,y2); flip at random so
        # both linedef orientations occur.
        if back >= 0 and rng.random() < 0.5:
            x1, y1, x2, y2, front, back = x2, y2, x1, y1, back, front
        walls.append((x1, y1, x2, y2))
        sectors.append((front, back))
        one_sided.append(back < 0)

    for r in range(R):
        for c in range(C):
            x0, y0 = c * room, r * room
            x1, y1 = x0 + room, y0 + room
            s = sid(r, c)
            if r == 0:
                add(x1, y0, x0, y0, s, -1)       # bottom edge, room above it
            if r == R - 1:
                add(x0, y1, x1, y1, s, -1)       # top edge
            if c == 0:
                add(x0, y0, x0, y1, s, -1)       # left edge
            if c == C - 1:
                add(x1, y1, x1, y0, s, -1)       # right edge
            if c + 1 < C:                          # shared vertical edge
                add(x1, y0, x1, y1, sid(r, c + 1), s)
            if r + 1 < R:                          # shared horizontal edge
                add(x0, y1, x1, y1, s, sid(r + 1, c))
    if spec.diagonals:
        for r in range(R):
            for c in range(C):
                x0, y0 = c * room, r * room
                x1, y1 = x0 + room, y0 + room
                s = sid(r, c)
                if rng.random() < 0.5:
                    walls.append((x0, y0, x1, y1))
                else:
                    walls.append((x0, y1, x1, y0))
                sectors.append((s, s))
                one_sided.append(False)

    walls = np.asarray(walls, dtype=np.float32)
    wall_sectors = np.asarray(sectors, dtype=np.int32)
    W = len(walls)
    self_ref = wall_sectors[:, 0] == wall_sectors[:, 1]

    T = spec.wall_textures
    F = spec.flats
    hmax = max(spec.tex_h, 64)
    wmax = max(spec.tex_w, 64)
    tex_atlas = np.zeros((T + F, hmax, wmax), dtype=np.uint8)
    tex_atlas[:T, : spec.tex_h, : spec.tex_w] = rng.integers(
        0, 256, size=(T, spec.tex_h, spec.tex_w), dtype=np.uint8)
    tex_atlas[T:, :64, :64] = rng.integers(0, 256, size=(F, 64, 64), dtype=np.uint8)
    tex_widths = np.asarray([spec.tex_w] * T + [64] * F, dtype=np.int32)
    tex_heights = np.asarray([spec.tex_h] * T + [64] * F, dtype=np.int32)

    side_textures = np.full((W, 2, 3), -1, dtype=np.int32)
    side_offsets = np.zeros((W, 2, 2), dtype=np.float32)
    for w in range(W):
        if self_ref[w]:
            continue
        if wall_sectors[w, 1] < 0:
            side_textures[w, 0, 0] = rng.integers(0, T)
        else:
            side_textures[w, :, 1] = rng.integers(0, T, size=2)
            side_textures[w, :, 2] = rng.integers(0, T, size=2)
        side_offsets[w] = rng.integers(0, 64, size=(2, 2)).astype(np.float32)

    if spec.mid_textures > 0:
        # drawn from a generator of their own so the other tables of a seed do not move
        mid_rng = np.random.default_rng(spec.seed + 1000)
        for w in range(W):
            if self_ref[w] or wall_sectors[w, 1] < 0:
                continue
            for side in range(2):
                if mid_rng.random() < spec.mid_textures:
                    side_textures[w, side, 0] = mid_rng.integers(0, T)

    sector_heights = np.stack(
        (
            rng.integers(0, spec.floor_max // 8 + 1, size=S) * 8,
            spec.ceil_lo + rng.integers(0, (spec.ceil_hi - spec.ceil_lo) // 8 + 1, size=S) * 8,
        ),
        axis=1,
    ).astype(np.float32)
    light_steps = (spec.light_hi - spec.light_lo) // 16 + 1
    sector_lights = (spec.light_lo + rng.integers(0, light_steps, size=S) * 16).astype(np.int16)
    sector_floor_tex = (T + rng.integers(0, F, size=S)).astype(np.int32)
    sector_ceil_tex = (T + rng.integers(0, F, size=S)).astype(np.int32)

    sector_edge_mask = np.zeros((S, W), dtype=np.bool_)
    for w in range(W):
        if self_ref[w]:
            continue
        for s in wall_sectors[w]:
            if s >= 0:
                sector_edge_mask[s, w] = True

    starts = np.zeros((spec.dolls + 1, 3), dtype=np.float32)
    starts[:, 0] = rng.uniform(32, C * spec.room - 32, size=spec.dolls + 1).round()
    starts[:, 1] = rng.uniform(32, R * spec.room - 32, size=spec.dolls + 1).round()
    starts[:, 2] = rng.integers(0, 8, size=spec.dolls + 1) * 45.0

    playpal = rng.integers(0, 256, size=(256, 3), dtype=np.uint8)
    idx = np.arange(256, dtype=np.int64)
    colormap = np.zeros((34, 256), dtype=np.uint8)
    for row in range(32):
        colormap[row] = (idx * (32 - row) // 32).astype(np.uint8)
    colormap[32] = (255 - idx).astype(np.uint8)
    colormap[33] = 0

    P = spec.sprite_patches
    spr_atlas, spr_opaque = _sprite_patches(rng, P, spec.spr_w, spec.spr_h)
    spr_widths = np.full(P, spec.spr_w, dtype=np.int32)
    spr_heights = np.full(P, spec.spr_h, dtype=np.int32)
    spr_left = (spec.spr_w // 2 + rng.integers(-2, 3, size=P)).astype(np.int32)
    spr_top = (spec.spr_h + rng.integers(-3, 1, size=P)).astype(np.int32)

    def ids(*shape):
        return rng.integers(0, P, size=shape).astype(np.int32)

    death_frames = 5
    additive = rng.integers(0, 256, size=(2, 256, 256), dtype=np.uint8)
    translucent = rng.integers(0, 256, size=(256, 256), dtype=np.uint8)

    if spec.weapon:
        Q, wh, ww = 12, 64, 96
        wpn_atlas = rng.integers(1, 256, size=(Q, wh, ww), dtype=np.uint8)
        holes = rng.random((Q, wh, ww)) < 0.1
        wpn_atlas[holes] = 0
        wpn_opaque = wpn_atlas != 0
        wpn_widths = rng.integers(48, ww + 1, size=Q).astype(np.int32)
        wpn_heights = rng.integers(40, wh + 1, size=Q).astype(np.int32)
        wpn_left = rng.integers(-160, -100, size=Q).astype(np.int32)
        wpn_top = rng.integers(-140, -100, size=Q).astype(np.int32)
        wpn_frame_ids = rng.integers(0, Q, size=(8, 2, WEAPON_TABLE_TICS)).astype(np.int32)
        wpn_flash_ids = rng.integers(-1, Q, size=(8, 2, WEAPON_TABLE_TICS)).astype(np.int32)
        wpn_flash_ids[:, :, 0] = -1
        wpn_flash_lights = np.zeros((8, 2, WEAPON_TABLE_TICS), dtype=np.int32)
    else:
        Q = 8
        wpn_atlas = np.zeros((Q, 1, 1), dtype=np.uint8)
        wpn_opaque = np.zeros((Q, 1, 1), dtype=np.bool_)
        wpn_widths = np.zeros(Q, dtype=np.int32)
        wpn_heights = np.zeros(Q, dtype=np.int32)
        wpn_left = np.zeros(Q, dtype=np.int32)
        wpn_top = np.zeros(Q, dtype=np.int32)
        wpn_frame_ids = np.broadcast_to(
            np.arange(8, dtype=np.int32)[:, None, None], (8, 2, WEAPON_TABLE_TICS)).copy()
        wpn_flash_ids = np.full((8, 2, WEAPON_TABLE_TICS), -1, dtype=np.int32)
        wpn_flash_lights = np.zeros((8, 2, WEAPON_TABLE_TICS), dtype=np.int32)

    hud_atlas = np.zeros((HUD_PATCHES, 32, 320), dtype=np.uint8)
    hud_opaque = np.zeros((HUD_PATCHES, 32, 320), dtype=np.bool_)
    hud_widths = np.zeros(HUD_PATCHES, dtype=np.int32)
    hud_heights = np.zeros(HUD_PATCHES, dtype=np.int32)
    hud_left = np.zeros(HUD_PATCHES, dtype=np.int32)
    hud_top = np.zeros(HUD_PATCHES, dtype=np.int32)
    if spec.hud:
        def patch(i, w, h, hole=0.0, left=0, top=0):
            data = rng.integers(0, 256, size=(h, w), dtype=np.uint8)
            hud_atlas[i, :h, :w] = data
            opaque = np.ones((h, w), dtype=np.bool_)
            if hole > 0:
                opaque &= rng.random((h, w)) >= hole
            hud_opaque[i, :h, :w] = opaque
            hud_widths[i], hud_heights[i] = w, h
            hud_left[i], hud_top[i] = left, top

        patch(0, 320, 32)                       # status bar
        patch(1, 40, 32, hole=0.1)              # arms panel
        for d in range(10):
            patch(2 + d, 14, 16, hole=0.3)      # large numerals
        patch(12, 14, 16, hole=0.3)             # percent sign
        for i in range(13, 28):
            patch(i, 24, 29, hole=0.1, left=-5, top=-2)   # straight faces
        for d in range(10):
            patch(28 + d, 4, 6, hole=0.2)       # small yellow numerals
        for i in range(38, 44):
            patch(i, 4, 6, hole=0.2)            # grey arms numerals
        for i in range(44, 70):
            patch(i, 24, 29, hole=0.1, left=-5, top=-2)   # other faces

    return Scene(
        walls=walls,
        wall_sectors=wall_sectors,
        side_textures=side_textures,
        side_offsets=side_offsets,
        sector_edge_mask=sector_edge_mask,
        sector_heights=sector_heights,
        sector_lights=sector_lights,
        sector_floor_tex=sector_floor_tex,
        sector_ceil_tex=sector_ceil_tex,
        player_starts=starts,
        tex_atlas=tex_atlas,
        tex_widths=tex_widths,
        tex_heights=tex_heights,
        playpal=playpal,
        colormap=colormap,
        spr_atlas=spr_atlas,
        spr_opaque=spr_opaque,
        spr_widths=spr_widths,
        spr_heights=spr_heights,
        spr_left=spr_left,
        spr_top=spr_top,
        enemy_walk_ids=ids(6, 4, 8),
        enemy_attack_ids=ids(6, 4, 8),
        enemy_pain_ids=ids(6, 8),
        enemy_death_ids=ids(6, death_frames),
        enemy_death_counts=np.full(6, death_frames, dtype=np.int32),
        enemy_death_durations=rng.integers(3, 9, size=(6, death_frames)).astype(np.int32),
        enemy_xdeath_ids=ids(6, death_frames),
        enemy_xdeath_counts=np.full(6, death_frames, dtype=np.int32),
        enemy_xdeath_durations=rng.integers(3, 9, size=(6, death_frames)).astype(np.int32),
        proj_flight_ids=ids(3, 2, 8),
        proj_explosion_ids=ids(3, 5),
        proj_explosion_counts=np.asarray((3, 5, 3), dtype=np.int32),
        proj_explosion_durations=np.asarray(
            ((8, 6, 4, 0, 0), (4, 4, 4, 4, 4), (6, 6, 6, 0, 0)), dtype=np.int32),
        fog_ids=ids(12),
        puff_ids=ids(4),
        static_ids=ids(20),
        additive_luts=additive,
        translucent_lut=translucent,
        wpn_atlas=wpn_atlas,
        wpn_opaque=wpn_opaque,
        wpn_widths=wpn_widths,
        wpn_heights=wpn_heights,
        wpn_left=wpn_left,
        wpn_top=wpn_top,
        wpn_frame_ids=wpn_frame_ids,
        wpn_flash_ids=wpn_flash_ids,
        wpn_flash_lights=wpn_flash_lights,
        hud_atlas=hud_atlas,
        hud_opaque=hud_opaque,
        hud_widths=hud_widths,
        hud_heights=hud_heights,
        hud_left=hud_left,
        hud_top=hud_top,
        meta=dict(_scene_meta(spec, None, P), **({"decals": _synthetic_decals(spec, colormap)} if spec.decals else {}),
                  **({"fragments": synthetic_fragments(walls, spec.splits, spec.seed + 4000)} if spec.splits > 0 else {})),
    )


def from_compiled_scenario(cs) -> Scene:
    """A Scene from the reference's ``CompiledScenario`` (src/gradoom/scenario.py:302-410), field
    by field; the defaults for absent optional fields are the ones the reference's device scene
    applies (src/gradoom/engine.py:869-1100).  Scenarios without the native renderer's assets
    (palette-indexed textures, raw sprites, status-bar patches) are refused."""

    def need(name):
        value = getattr(cs, name, None)
        if value is None:
            raise ValueError(f"the compiled scenario lacks {name!r}, which the native render path needs")
        return np.asarray(value)

    def maybe(name, default):
        value = getattr(cs, name, None)
        return np.asarray(default if value is None else value)

    # every line is one fragment unless a node builder split it (src/gradoom/scenario.py:420-455)
    fragment_mask = getattr(cs, "wall_projection_fragment_mask", None)
    fragments = getattr(cs, "wall_projection_fragments_fixed", None)
    if (fragment_mask is None) != (fragments is None):
        raise ValueError("wall projection fragments and their mask must be provided together")
    split_lines = {}
    if fragments is not None:
        fragments, fragment_mask = np.asarray(fragments), np.asarray(fragment_mask).astype(bool)
        if fragments.shape[:2] != fragment_mask.shape or fragments.shape[2:] != (4,):
            raise ValueError("invalid wall projection fragment arrays")
        for line in np.flatnonzero(fragment_mask.sum(axis=1) > 1):
            split_lines[int(line)] = fragments[line][fragment_mask[line]].astype(np.int64)
    spr_atlas = need("raw_sprite_atlas")
    last_sprite = max(len(spr_atlas) - 1, 0)
    wpn_atlas = getattr(cs, "native_weapon_patch_atlas", None)
    if wpn_atlas is None:
        wpn = {"atlas": np.zeros((1, 1, 1), np.uint8), "opaque": np.zeros((1, 1, 1), bool),
               "widths": np.zeros(1, np.int32), "heights": np.zeros(1, np.int32), "left": np.zeros(1, np.int32),
               "top": np.zeros(1, np.int32)}
    else:
        wpn = {"atlas": np.asarray(wpn_atlas), "opaque": need("native_weapon_patch_opaque"),
               "widths": need("native_weapon_patch_widths"), "heights": need("native_weapon_patch_heights"),
               "left": need("native_weapon_patch_left_offsets"), "top": need("native_weapon_patch_top_offsets")}
    meta = {}
    item_types = np.asarray(getattr(cs, "item_types", np.empty(0, np.int32)))
    if len(item_types):
        meta["items"] = {"spawns": np.asarray(cs.item_spawns, dtype=np.float32), "types": item_types.astype(np.int32),
                         "anim_ids": maybe("raw_item_animation_sprite_ids", np.zeros(8, np.int32)).astype(np.int32)}
    if split_lines:
        meta["fragments"] = split_lines
    if getattr(cs, "bullet_decal_atlas", None) is not None:
        meta["decals"] = {"atlas": need("bullet_decal_atlas").astype(np.uint8),
                          "heights": need("bullet_decal_heights").astype(np.int32),
                          "left": need("bullet_decal_left_offsets").astype(np.int32),
                          "top": need("bullet_decal_top_offsets").astype(np.int32),
                          "opacity_lut": need("bullet_decal_opacity_lut").astype(np.uint8),
                          "black_lut": need("bullet_decal_black_lut").astype(np.uint8)}
    return Scene(
        walls=need("wall_segments").astype(np.float32), wall_sectors=need("wall_sectors").astype(np.int32),
        side_textures=need("wall_side_texture_ids").astype(np.int32),
        side_offsets=need("wall_side_texture_offsets").astype(np.float32),
        sector_edge_mask=need("sector_edge_mask").astype(np.bool_),
        sector_heights=need("sector_heights").astype(np.float32), sector_lights=need("sector_lights").astype(np.int16),
        sector_floor_tex=need("sector_floor_texture_ids").astype(np.int32),
        sector_ceil_tex=need("sector_ceiling_texture_ids").astype(np.int32),
        player_starts=need("player_starts").astype(np.float32),
        tex_atlas=need("texture_index_atlas").astype(np.uint8), tex_widths=need("texture_widths").astype(np.int32),
        tex_heights=need("texture_heights").astype(np.int32), playpal=need("playpal").astype(np.uint8),
        colormap=maybe("colormap", np.broadcast_to(np.arange(256, dtype=np.uint8), (34, 256))).astype(np.uint8),
        spr_atlas=spr_atlas.astype(np.uint8), spr_opaque=need("raw_sprite_opaque").astype(np.bool_),
        spr_widths=need("raw_sprite_widths").astype(np.int32), spr_heights=need("raw_sprite_heights").astype(np.int32),
        spr_left=need("raw_sprite_left_offsets").astype(np.int32), spr_top=need("raw_sprite_top_offsets").astype(np.int32),
        enemy_walk_ids=need("enemy_walk_sprite_ids").astype(np.int32),
        enemy_attack_ids=need("enemy_attack_sprite_ids").astype(np.int32),
        enemy_pain_ids=need("enemy_pain_sprite_ids").astype(np.int32),
        enemy_death_ids=need("enemy_death_sprite_ids").astype(np.int32),
        enemy_death_counts=need("enemy_death_frame_counts").astype(np.int32),
        enemy_death_durations=need("enemy_death_frame_durations").astype(np.int32),
        enemy_xdeath_ids=need("enemy_xdeath_sprite_ids").astype(np.int32),
        enemy_xdeath_counts=need("enemy_xdeath_frame_counts").astype(np.int32),
        enemy_xdeath_durations=need("enemy_xdeath_frame_durations").astype(np.int32),
        proj_flight_ids=need("raw_projectile_flight_sprite_ids").astype(np.int32),
        proj_explosion_ids=need("raw_projectile_explosion_sprite_ids").astype(np.int32),
        proj_explosion_counts=need("projectile_explosion_frame_counts").astype(np.int32),
        proj_explosion_durations=need("projectile_explosion_frame_durations").astype(np.int32),
        fog_ids=need("raw_teleport_fog_sprite_ids").astype(np.int32), puff_ids=need("raw_bullet_puff_sprite_ids").astype(np.int32),
        static_ids=maybe("raw_static_sprite_ids", [min(i, last_sprite) for i in range(6, 26)]).astype(np.int32),
        additive_luts=need("projectile_additive_luts").astype(np.uint8),
        translucent_lut=need("sprite_translucent_lut").astype(np.uint8),
        wpn_atlas=wpn["atlas"].astype(np.uint8), wpn_opaque=wpn["opaque"].astype(np.bool_),
        wpn_widths=wpn["widths"].astype(np.int32), wpn_heights=wpn["heights"].astype(np.int32),
        wpn_left=wpn["left"].astype(np.int32), wpn_top=wpn["top"].astype(np.int32),
        wpn_frame_ids=need("native_weapon_frame_ids").astype(np.int32),
        wpn_flash_ids=need("native_weapon_flash_ids").astype(np.int32),
        wpn_flash_lights=need("native_weapon_flash_lights").astype(np.int32),
        hud_atlas=need("hud_patch_atlas").astype(np.uint8), hud_opaque=need("hud_patch_opaque").astype(np.bool_),
        hud_widths=need("hud_patch_widths").astype(np.int32), hud_heights=need("hud_patch_heights").astype(np.int32),
        hud_left=need("hud_patch_left_offsets").astype(np.int32), hud_top=need("hud_patch_top_offsets").astype(np.int32),
        meta=meta,
    )


# ---------------------------------------------------------------------------
# Packing a Scene into the device blob (layout: include/gradoom_b200_layout.h)
# ---------------------------------------------------------------------------

GD_MAGIC = 0x4744424C
GD_VERSION = 11
GD_HDR_WORDS = 160
GD_HDR_SECTION0 = 48

_HEADER_WORDS = (
    "MAGIC VERSION BYTES WALLS SECTORS VERTICES TEXTURES TEX_H TEX_W SPRITES SPR_H SPR_W "
    "WPN_PATCHES WPN_H WPN_W WPN_TICS STARTS DEATH_FRAMES XDEATH_FRAMES BLOCKING NB_DIRECT "
    "WPN_AVAILABLE HUD_PATCHES UNSUPPORTED SEC_WALLS_N VTX_WALLS_N MASKED_WALLS_N FLOOR_GROUPS CEIL_GROUPS ITEMS "
    "DECALS DECAL_H DECAL_W FRAGMENTS"
).split()
H = {name: i for i, name in enumerate(_HEADER_WORDS)}

_SECTIONS = (
    "WALLS WALL_SECTORS WALL_LEN SIDE_TEX SIDE_OFF WALL_VTX VTX_OFF VTX_WALLS NB_DIRECT NB_OFF "
    "NB_IDX NB_FLAGS SB_START_OFF SB_START_IDX SB_END_OFF SB_END_IDX SECTOR_F SECTOR_I SEC_OFF "
    "SEC_WALLS EDGE_OFF EDGE_WALLS BLOCKING TEX_INFO TEX_ATLAS PLAYPAL COLORMAP SPR_INFO "
    "SPR_ATLAS SPR_POST ENEMY_WALK ENEMY_ATTACK ENEMY_PAIN DEATH_IDS DEATH_COUNTS DEATH_ENDS "
    "XDEATH_IDS XDEATH_COUNTS XDEATH_ENDS PROJ_FLIGHT PROJ_EXPL_IDS PROJ_EXPL_COUNTS "
    "PROJ_EXPL_ENDS PROJ_EXPL_TOTAL FOG_IDS PUFF_IDS STATIC_IDS ADD_LUT TRANS_LUT WPN_INFO "
    "WPN_ATLAS WPN_OPAQUE WPN_FRAME_IDS WPN_FLASH_IDS WPN_FLASH_LIGHTS HUD_INFO HUD_ATLAS "
    "HUD_OPAQUE FINESINE FINETAN STARTS RAY_OFFSETS RAY_COSCORR TEX_ATLAS_COL SECTOR_BBOX "
    "MASKED_WALLS DAMAGE_ALPHA FLOOR_GROUP_H FLOOR_GROUP_OFF FLOOR_GROUP_SEC CEIL_GROUP_H CEIL_GROUP_OFF "
    "CEIL_GROUP_SEC ITEM_POS ITEM_INFO ITEM_ANIM DECAL_INFO DECAL_ATLAS DECAL_OPACITY DECAL_BLACK WALL_FINE "
    "FRAG_OFF FRAG_FIXED"
).split()
SEC = {name: i for i, name in enumerate(_SECTIONS)}

FIXED_UNIT = 1 << 16
FINE_ANGLES = 8192


def wall_fine_angles(walls: np.ndarray) -> np.ndarray:
    """(W, 2) fine-angle index of each wall's direction as seen from side 0 and from side 1
    (the direction reversed): atan2 of the float32 wall vector, wrapped to [0, 2 pi) and quantised
    to 8192 steps (src/gradoom/engine.py:2153-2165, 13818-13830).  Evaluated with torch's float32
    kernels, the arithmetic the reference itself runs, so that a direction on a step boundary
    (every multiple of 45 degrees is one) lands on the same side."""

    import math
    import torch

    w = torch.from_numpy(np.ascontiguousarray(walls, dtype=np.float32))
    vec = w[:, 2:] - w[:, :2]
    out = np.zeros((len(walls), 2), dtype=np.int32)
    for side in (0, 1):
        oriented = vec if side == 0 else -vec
        angle = torch.atan2(oriented[:, 1], oriented[:, 0])
        index = torch.floor(torch.remainder(angle, 2.0 * math.pi) * (FINE_ANGLES / (2.0 * math.pi))).to(torch.int64)
        out[:, side] = (index & (FINE_ANGLES - 1)).numpy()
    return out


def fine_sine_table() -> np.ndarray:
    """16.16 sine table of 8192 fine angles (definition:
    src/gradoom/engine.py:309-320): first quadrant truncated, mirrored, negated,
    with the two extrema forced to +-1.0."""

    q = FINE_ANGLES // 4
    first = np.trunc(np.sin(np.arange(q, dtype=np.float64) * (2.0 * np.pi / FINE_ANGLES))
                     * FIXED_UNIT).astype(np.int64)
    table = np.concatenate((first, first[::-1]))
    table = np.concatenate((table, -table))
    table[q] = FIXED_UNIT
    table[3 * q] = -FIXED_UNIT
    return table.astype(np.int32)


def fine_tangent_table() -> np.ndarray:
    """16.16 tangent table of 4096 entries (src/gradoom/engine.py:323-328)."""

    half = FINE_ANGLES // 2
    phase = (np.arange(half, dtype=np.float64) - FINE_ANGLES // 4) * (2.0 * np.pi / FINE_ANGLES)
    phase[0] += np.pi / FINE_ANGLES
    return np.trunc(np.tan(phase) * FIXED_UNIT + 0.5).astype(np.int64).astype(np.int32)


def sector_at(scene: Scene, x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """First sector whose edge set has odd crossing parity for a +x ray, else 0.

    float32 arithmetic in the reference's order (src/gradoom/engine.py:9598-9617).
    """

    x = np.asarray(x, dtype=np.float32).reshape(-1)
    y = np.asarray(y, dtype=np.float32).reshape(-1)
    e = scene.walls.astype(np.float32)
    x1, y1, x2, y2 = e[:, 0], e[:, 1], e[:, 2], e[:, 3]
    px, py = x[:, None], y[:, None]
    crosses = (y1 > py) != (y2 > py)
    dy = y2 - y1
    safe = np.where(np.abs(dy) < np.float32(1e-6), np.float32(1), dy).astype(np.float32)
    crossing = (x1 + ((py - y1) * (x2 - x1)).astype(np.float32) / safe).astype(np.float32)
    hit = crosses & (px < crossing)
    parity = (hit[:, None, :] & scene.sector_edge_mask[None, :, :]).sum(axis=2) % 2
    return np.argmax(parity, axis=1).astype(np.int64)


def _csr(lists):
    off = np.zeros(len(lists) + 1, dtype=np.int32)
    for i, l in enumerate(lists):
        off[i + 1] = off[i] + len(l)
    idx = np.asarray([v for l in lists for v in l], dtype=np.int32)
    if idx.size == 0:
        idx = np.zeros(1, dtype=np.int32)
    return off, idx


def ray_tables():
    """Per-column ray angle offsets of the flat fallback and their cosines, in
    float32 as the host framework evaluates them
    (src/gradoom/engine.py:2050-2054, 10967)."""

    import torch

    columns = torch.arange(320, dtype=torch.float32) - 320 / 2.0
    offsets = -torch.atan(columns / (320 / 2.0))
    return offsets.numpy().copy(), torch.cos(offsets).numpy().copy()


def pack_scene(scene: Scene, ray_table_override=None) -> np.ndarray:
    """Serialise a Scene plus its static topology tables into one byte blob.

    ``ray_table_override`` supplies ``(offsets, cosines)`` recorded elsewhere, so
    a fixture generated on one machine replays bit-identically on another.
    """

    import torch  # deg2rad in float32 exactly as the host framework computes it

    walls = np.ascontiguousarray(scene.walls, dtype=np.float32) + np.float32(0.0)
    sectors = np.ascontiguousarray(scene.wall_sectors, dtype=np.int32)
    W, S = len(walls), scene.num_sectors
    one_sided = sectors[:, 1] < 0
    unsupported = 0

    def height_groups(values, descending):
        """Sectors grouped by plane height, nearest plane first for a viewer between
        the planes: (heights, CSR offsets, sector indices ascending inside a group)."""

        values = np.asarray(values, dtype=np.float32)
        heights = np.unique(values)
        if descending:
            heights = heights[::-1]
        members = [np.flatnonzero(values == h).astype(np.int32) for h in heights]
        offsets = np.concatenate(([0], np.cumsum([len(m) for m in members]))).astype(np.int32)
        return np.ascontiguousarray(heights, dtype=np.float32), offsets, np.concatenate(members).astype(np.int32)

    floor_groups = height_groups(scene.sector_heights[:, 0], descending=True)
    ceil_groups = height_groups(scene.sector_heights[:, 1], descending=False)
    # red-flash alpha per damage count (src/gradoom/engine.py:2016, 15393); a scene built from an
    # engine carries the engine's table in meta["damage_alpha"], synthetic scenes use a plain ramp
    damage_alpha = np.asarray(scene.meta.get("damage_alpha", np.minimum(np.arange(114) * 2.0, 226.0)),
                              dtype=np.float32)
    assert damage_alpha.shape == (114,)
    # two-sided lines with a middle (masked) texture on either side, ascending
    masked_walls = np.flatnonzero((~one_sided) & (scene.side_textures[:, :, 0].max(axis=1) >= 0)).astype(np.int32)

    dx = walls[:, 2] - walls[:, 0]
    dy = walls[:, 3] - walls[:, 1]
    wall_len = np.floor(np.sqrt(np.square(dx) + np.square(dy)) + np.float32(0.5)).astype(np.float32)

    pts = walls.reshape(-1, 2)
    verts, inverse = np.unique(pts, axis=0, return_inverse=True)
    wall_vtx = inverse.reshape(W, 2).astype(np.int32)
    V = len(verts)
    vtx_lists = [[] for _ in range(V)]
    for w in range(W):
        for e in range(2):
            if w not in vtx_lists[wall_vtx[w, e]]:
                vtx_lists[wall_vtx[w, e]].append(w)
    vtx_off, vtx_walls = _csr(vtx_lists)

    same_pair = ((sectors[:, None, 0] == sectors[None, :, 0]) & (sectors[:, None, 1] == sectors[None, :, 1])) | (
        (sectors[:, None, 0] == sectors[None, :, 1]) & (sectors[:, None, 1] == sectors[None, :, 0]))
    v0, v1 = wall_vtx[:, 0], wall_vtx[:, 1]
    shares_start = (v0[:, None] == v0[None, :]) | (v0[:, None] == v1[None, :])
    shares_end = (v1[:, None] == v0[None, :]) | (v1[:, None] == v1[None, :])
    eye = np.eye(W, dtype=np.bool_)
    nb_mask = same_pair & (shares_start | shares_end) & ~eye
    nb_lists, nb_flag_lists = [], []
    for w in range(W):
        idx = np.flatnonzero(nb_mask[w])
        nb_lists.append(idx.tolist())
        nb_flag_lists.append((shares_start[w, idx].astype(np.int32)
                              + 2 * shares_end[w, idx].astype(np.int32)).tolist())
    nb_off, nb_idx = _csr(nb_lists)
    _, nb_flags = _csr(nb_flag_lists)
    start_counts = np.asarray([sum(f & 1 for f in fl) for fl in nb_flag_lists])
    end_counts = np.asarray([sum((f >> 1) & 1 for f in fl) for fl in nb_flag_lists])
    nb_direct_ok = int(np.all(start_counts <= 1) and np.all(end_counts <= 1))
    nb_direct = np.full((W, 4), -1, dtype=np.int32)
    nb_direct[:, 2:] = 0
    for w in range(W):
        # slot of the first neighbour sharing the start / the end (0 when none),
        # and the neighbour stored in that slot (the wall itself when the list is empty).
        fl = nb_flag_lists[w]
        s_slot = next((k for k, f in enumerate(fl) if f & 1), 0)
        e_slot = next((k for k, f in enumerate(fl) if f & 2), 0)
        nb_direct[w, 2], nb_direct[w, 3] = s_slot, e_slot
        nb_direct[w, 0] = nb_lists[w][s_slot] if start_counts[w] > 0 else -1
        nb_direct[w, 1] = nb_lists[w][e_slot] if end_counts[w] > 0 else -1

    same_solid = sectors[:, None, 0] == sectors[None, :, 0]
    adjacency = (shares_start | shares_end) & one_sided[:, None] & one_sided[None, :] & same_solid & ~eye
    sel_solid = (sectors[:, None, 0] == sectors[None, :, 0]) | (sectors[:, None, 1] == sectors[None, :, 0])
    sb_start = ((shares_start & one_sided[None, :] & sel_solid).astype(np.int32) @ adjacency.astype(np.int32)) > 0
    sb_end = ((shares_end & one_sided[None, :] & sel_solid).astype(np.int32) @ adjacency.astype(np.int32)) > 0
    sb_start_off, sb_start_idx = _csr([np.flatnonzero(sb_start[w]).tolist() for w in range(W)])
    sb_end_off, sb_end_idx = _csr([np.flatnonzero(sb_end[w]).tolist() for w in range(W)])

    sec_lists = [np.flatnonzero((sectors[:, 0] == s) | (sectors[:, 1] == s)).tolist() for s in range(S)]
    sec_off, sec_walls = _csr(sec_lists)
    edge_off, edge_walls = _csr([np.flatnonzero(scene.sector_edge_mask[s]).tolist() for s in range(S)])
    blocking = np.flatnonzero(one_sided).astype(np.int32)
    if blocking.size == 0:
        blocking = np.zeros(1, dtype=np.int32)
        unsupported |= 2

    T = len(scene.tex_atlas)
    tex_info = np.zeros((T, 4), dtype=np.int32)
    tex_info[:, 0] = scene.tex_widths
    tex_info[:, 1] = scene.tex_heights
    tex_info[:, 2] = np.floor(np.log2(scene.tex_widths.astype(np.float32))).astype(np.int32)
    tex_info[:, 3] = np.floor(np.log2(scene.tex_heights.astype(np.float32))).astype(np.int32)

    P = len(scene.spr_atlas)
    spr_info = np.stack((scene.spr_widths, scene.spr_heights, scene.spr_left, scene.spr_top),
                        axis=1).astype(np.int32)
    opaque = scene.spr_opaque.astype(np.bool_)
    prior = np.concatenate((np.zeros_like(opaque[:, :1]), opaque[:, :-1]), axis=1)
    starts_post = opaque & ~prior
    rows = np.arange(opaque.shape[1], dtype=np.int64)[None, :, None]
    post_top = np.maximum.accumulate(np.where(starts_post, rows, 0), axis=1)
    if opaque.shape[1] >= 255:
        unsupported |= 4
    spr_post = np.where(opaque, post_top, 255).astype(np.uint8)

    def ends(durations):
        return np.cumsum(durations.astype(np.int64), axis=-1).astype(np.int32)

    start_sectors = sector_at(scene, scene.player_starts[:, 0], scene.player_starts[:, 1])
    starts = np.zeros((len(scene.player_starts), 4), dtype=np.float32)
    starts[:, 0:2] = scene.player_starts[:, 0:2]
    starts[:, 2] = torch.deg2rad(torch.as_tensor(scene.player_starts[:, 2].astype(np.float32))).numpy()
    starts[:, 3] = scene.sector_heights[start_sectors, 0]

    ray_offsets, ray_coscorr = ray_tables() if ray_table_override is None else ray_table_override
    sector_i = np.zeros((S, 4), dtype=np.int32)
    sector_i[:, 0] = scene.sector_lights
    sector_i[:, 1] = scene.sector_floor_tex
    sector_i[:, 2] = scene.sector_ceil_tex

    bbox = np.zeros((S, 4), dtype=np.float32)
    for s_ in range(S):
        ew = np.flatnonzero(scene.sector_edge_mask[s_])
        if len(ew) == 0:
            bbox[s_] = (1.0, 0.0, 1.0, 0.0)
            continue
        ex = walls[ew][:, (0, 2)]
        ey = walls[ew][:, (1, 3)]
        bbox[s_] = (ex.min(), ex.max(), ey.min(), ey.max())
        degree = np.bincount(wall_vtx[ew].reshape(-1), minlength=V)
        sector_i[s_, 3] = int(np.all(degree % 2 == 0))

    def info4(a, b, c, d):
        return np.stack((a, b, c, d), axis=1).astype(np.int32)

    # Projection fragments of lines a node builder split (src/gradoom/scenario.py:420-455,
    # engine.py:745-767): an optional meta["fragments"] = {wall index: (F,4) int64 16.16 endpoints,
    # in order}.  Lines absent from it, or with a single fragment, project as a whole.
    frag_off = np.zeros(W + 1, dtype=np.int32)
    frag_rows = []
    for w_, pieces in sorted((scene.meta.get("fragments") or {}).items()):
        pieces = np.asarray(pieces, dtype=np.int64).reshape(-1, 4)
        if not 0 <= w_ < W:
            raise ValueError(f"fragments given for line {w_}, the scene has {W}")
        if len(pieces) > 1:
            frag_off[w_ + 1] = len(pieces)
            frag_rows.append(pieces)
    frag_off = np.cumsum(frag_off).astype(np.int32)
    n_fragments = int(frag_off[-1])
    frag_fixed = (np.concatenate(frag_rows) if frag_rows else np.zeros((1, 4), dtype=np.int64)).astype(np.int32)

    # Bullet-chip decals (src/gradoom/scenario.py:280-300, engine.py:1038-1068): an optional
    # meta["decals"] = {"atlas": (V,h,w) u8, "heights", "left", "top": (V,), "opacity_lut": (32,256),
    # "black_lut": (65,256)}.  Without it the decal layer draws nothing, as the reference's zero atlas.
    decals = scene.meta.get("decals")
    n_decals = 0 if decals is None else len(decals["heights"])
    decal_atlas = np.zeros((1, 1, 1), dtype=np.uint8) if decals is None else np.asarray(decals["atlas"], dtype=np.uint8)
    decal_info = np.zeros((max(n_decals, 1), 4), dtype=np.int32)
    decal_opacity = np.zeros((32, 256), dtype=np.uint8)
    decal_black = np.broadcast_to(np.arange(256, dtype=np.uint8), (65, 256)).copy()
    if n_decals:
        if decal_atlas.ndim != 3 or len(decal_atlas) != n_decals:
            raise ValueError("the decal atlas must hold one (h, w) slice per chip variant")
        decal_info[:, 0] = decals["heights"]
        decal_info[:, 1] = decals["left"]
        decal_info[:, 2] = decals["top"]
        decal_opacity = np.asarray(decals["opacity_lut"], dtype=np.uint8).reshape(32, 256)
        decal_black = np.asarray(decals["black_lut"], dtype=np.uint8).reshape(65, 256)

    # Map items (pickups placed by the map; src/gradoom/engine.py:1084-1088, 2077-2081): an optional
    # meta["items"] = {"spawns": (I,3) x y z-above-floor, "types": (I,) editor ids, "anim_ids": (8,)}.
    items = scene.meta.get("items")
    n_items = 0 if items is None else len(items["types"])
    item_pos = np.zeros((max(n_items, 1), 4), dtype=np.float32)
    item_info = np.zeros((max(n_items, 1), 2), dtype=np.int32)
    item_anim = np.zeros(8, dtype=np.int32)
    if n_items:
        spawns = np.asarray(items["spawns"], dtype=np.float32)
        types = np.asarray(items["types"], dtype=np.int32)
        item_pos[:, 0:2] = spawns[:, 0:2]
        item_pos[:, 2] = scene.sector_heights[sector_at(scene, spawns[:, 0], spawns[:, 1]), 0] + spawns[:, 2]
        item_info[:, 0] = types
        for i, t in enumerate(types.tolist()):
            if t not in ITEM_SPRITE_INDEX:
                raise ValueError(f"unsupported item type {t}")
            item_info[i, 1] = scene.static_ids[ITEM_SPRITE_INDEX[t] - 6]
        item_anim[:] = np.asarray(items.get("anim_ids", np.zeros(8)), dtype=np.int32)

    sections = {
        "WALLS": walls,
        "WALL_SECTORS": sectors,
        "WALL_LEN": wall_len,
        "SIDE_TEX": scene.side_textures.astype(np.int32),
        "SIDE_OFF": scene.side_offsets.astype(np.float32),
        "WALL_VTX": wall_vtx,
        "VTX_OFF": vtx_off,
        "VTX_WALLS": vtx_walls,
        "NB_DIRECT": nb_direct,
        "NB_OFF": nb_off,
        "NB_IDX": nb_idx,
        "NB_FLAGS": nb_flags,
        "SB_START_OFF": sb_start_off,
        "SB_START_IDX": sb_start_idx,
        "SB_END_OFF": sb_end_off,
        "SB_END_IDX": sb_end_idx,
        "SECTOR_F": scene.sector_heights.astype(np.float32),
        "SECTOR_I": sector_i,
        "SEC_OFF": sec_off,
        "SEC_WALLS": sec_walls,
        "EDGE_OFF": edge_off,
        "EDGE_WALLS": edge_walls,
        "BLOCKING": blocking,
        "TEX_INFO": tex_info,
        "TEX_ATLAS": scene.tex_atlas.astype(np.uint8),
        "PLAYPAL": scene.playpal.astype(np.uint8),
        "COLORMAP": scene.colormap.astype(np.uint8),
        "SPR_INFO": spr_info,
        "SPR_ATLAS": scene.spr_atlas.astype(np.uint8),
        "SPR_POST": spr_post,
        "ENEMY_WALK": scene.enemy_walk_ids.astype(np.int32),
        "ENEMY_ATTACK": scene.enemy_attack_ids.astype(np.int32),
        "ENEMY_PAIN": scene.enemy_pain_ids.astype(np.int32),
        "DEATH_IDS": scene.enemy_death_ids.astype(np.int32),
        "DEATH_COUNTS": scene.enemy_death_counts.astype(np.int32),
        "DEATH_ENDS": ends(scene.enemy_death_durations),
        "XDEATH_IDS": scene.enemy_xdeath_ids.astype(np.int32),
        "XDEATH_COUNTS": scene.enemy_xdeath_counts.astype(np.int32),
        "XDEATH_ENDS": ends(scene.enemy_xdeath_durations),
        "PROJ_FLIGHT": scene.proj_flight_ids.astype(np.int32),
        "PROJ_EXPL_IDS": scene.proj_explosion_ids.astype(np.int32),
        "PROJ_EXPL_COUNTS": scene.proj_explosion_counts.astype(np.int32),
        "PROJ_EXPL_ENDS": ends(scene.proj_explosion_durations),
        "PROJ_EXPL_TOTAL": scene.proj_explosion_durations.sum(axis=1).astype(np.int32),
        "FOG_IDS": scene.fog_ids.astype(np.int32),
        "PUFF_IDS": scene.puff_ids.astype(np.int32),
        "STATIC_IDS": scene.static_ids.astype(np.int32),
        "ADD_LUT": scene.additive_luts.astype(np.uint8),
        "TRANS_LUT": scene.translucent_lut.astype(np.uint8),
        "WPN_INFO": info4(scene.wpn_widths, scene.wpn_heights, scene.wpn_left, scene.wpn_top),
        "WPN_ATLAS": scene.wpn_atlas.astype(np.uint8),
        "WPN_OPAQUE": scene.wpn_opaque.astype(np.uint8),
        "WPN_FRAME_IDS": scene.wpn_frame_ids.astype(np.int32),
        "WPN_FLASH_IDS": scene.wpn_flash_ids.astype(np.int32),
        "WPN_FLASH_LIGHTS": scene.wpn_flash_lights.astype(np.int32),
        "HUD_INFO": info4(scene.hud_widths, scene.hud_heights, scene.hud_left, scene.hud_top),
        "HUD_ATLAS": scene.hud_atlas.astype(np.uint8),
        "HUD_OPAQUE": scene.hud_opaque.astype(np.uint8),
        "FINESINE": fine_sine_table(),
        "FINETAN": fine_tangent_table(),
        "STARTS": starts,
        "RAY_OFFSETS": np.asarray(ray_offsets, dtype=np.float32),
        "RAY_COSCORR": np.asarray(ray_coscorr, dtype=np.float32),
        "TEX_ATLAS_COL": np.ascontiguousarray(scene.tex_atlas.astype(np.uint8).transpose(0, 2, 1)),
        "SECTOR_BBOX": bbox,
        "MASKED_WALLS": masked_walls if masked_walls.size else np.zeros(1, dtype=np.int32),
        "DAMAGE_ALPHA": damage_alpha,
        "FLOOR_GROUP_H": floor_groups[0], "FLOOR_GROUP_OFF": floor_groups[1], "FLOOR_GROUP_SEC": floor_groups[2],
        "CEIL_GROUP_H": ceil_groups[0], "CEIL_GROUP_OFF": ceil_groups[1], "CEIL_GROUP_SEC": ceil_groups[2],
        "ITEM_POS": item_pos, "ITEM_INFO": item_info, "ITEM_ANIM": item_anim,
        "DECAL_INFO": decal_info, "DECAL_ATLAS": decal_atlas, "DECAL_OPACITY": decal_opacity,
        "DECAL_BLACK": decal_black, "WALL_FINE": wall_fine_angles(walls),
        "FRAG_OFF": frag_off, "FRAG_FIXED": frag_fixed,
    }
    assert set(sections) == set(SEC), set(SEC) ^ set(sections)

    header = np.zeros(GD_HDR_WORDS, dtype=np.int32)
    chunks = []
    cursor = GD_HDR_WORDS * 4
    for name in _SECTIONS:
        data = np.ascontiguousarray(sections[name]).view(np.uint8).reshape(-1)
        pad = (-cursor) % 128        # a texture column of 128 texels then lies in one 128-byte line
        if pad:
            chunks.append(np.zeros(pad, dtype=np.uint8))
            cursor += pad
        header[GD_HDR_SECTION0 + SEC[name]] = cursor
        chunks.append(data)
        cursor += data.size
    pad = (-cursor) % 16
    if pad:
        chunks.append(np.zeros(pad, dtype=np.uint8))
        cursor += pad

    header[H["MAGIC"]] = GD_MAGIC
    header[H["VERSION"]] = GD_VERSION
    header[H["BYTES"]] = cursor
    header[H["WALLS"]] = W
    header[H["SECTORS"]] = S
    header[H["VERTICES"]] = V
    header[H["TEXTURES"]] = T
    header[H["TEX_H"]] = scene.tex_atlas.shape[1]
    header[H["TEX_W"]] = scene.tex_atlas.shape[2]
    header[H["SPRITES"]] = P
    header[H["SPR_H"]] = scene.spr_atlas.shape[1]
    header[H["SPR_W"]] = scene.spr_atlas.shape[2]
    header[H["WPN_PATCHES"]] = len(scene.wpn_atlas)
    header[H["WPN_H"]] = scene.wpn_atlas.shape[1]
    header[H["WPN_W"]] = scene.wpn_atlas.shape[2]
    header[H["WPN_TICS"]] = scene.wpn_frame_ids.shape[2]
    header[H["STARTS"]] = len(scene.player_starts)
    header[H["DEATH_FRAMES"]] = scene.enemy_death_ids.shape[1]
    header[H["XDEATH_FRAMES"]] = scene.enemy_xdeath_ids.shape[1]
    header[H["BLOCKING"]] = int(one_sided.sum())
    header[H["NB_DIRECT"]] = nb_direct_ok
    header[H["WPN_AVAILABLE"]] = int(scene.wpn_widths.max() > 0)
    header[H["HUD_PATCHES"]] = len(scene.hud_atlas)
    header[H["UNSUPPORTED"]] = unsupported
    header[H["SEC_WALLS_N"]] = int(sec_off[-1])
    header[H["VTX_WALLS_N"]] = int(vtx_off[-1])
    header[H["MASKED_WALLS_N"]] = int(masked_walls.size)
    header[H["FLOOR_GROUPS"]] = int(floor_groups[0].size)
    header[H["CEIL_GROUPS"]] = int(ceil_groups[0].size)
    header[H["ITEMS"]] = n_items
    header[H["DECALS"]] = n_decals
    header[H["FRAGMENTS"]] = n_fragments
    header[H["DECAL_H"]] = decal_atlas.shape[1]
    header[H["DECAL_W"]] = decal_atlas.shape[2]
    blob = np.concatenate([header.view(np.uint8)] + chunks)
    assert blob.size == cursor
    return blob
