"""Seeded synthetic lane states and a minimal lane stepper.

The renderer's inputs normally come from a game-dynamics engine, which is
outside this package.  For throughput runs and for tests that must not depend
on that engine, this module draws lane states directly: player poses uniform
over the map's rooms, `k` things per lane at uniform room positions, weapon and
status-bar scalars in their usual ranges.  ``advance`` then turns and moves the
players between renders so successive frames differ.  None of this claims
parity with the reference's dynamics; it only produces valid render inputs.
"""

from __future__ import annotations

import numpy as np

from . import scene as gdscene
from . import state as gdstate

FIXED_UNIT = 1 << 16
VIEW_HEIGHT = 41.0


def random_lanes(sc: gdscene.Scene, n: int, k_things: int, seed: int, max_things: int | None = None):
    """Return ``(lanes (n,32) int32, things (n,K,4) int32)`` as numpy arrays."""

    rng = np.random.default_rng(seed)
    spec = sc.meta["spec"]
    width, height = spec.cols * spec.room, spec.rows * spec.room
    lanes = np.zeros((n, gdstate.LANE_WORDS), dtype=np.int32)
    lf = lanes.view(np.float32)

    x_fixed = np.round(rng.uniform(24.0, width - 24.0, size=n) * FIXED_UNIT).astype(np.int64)
    y_fixed = np.round(rng.uniform(24.0, height - 24.0, size=n) * FIXED_UNIT).astype(np.int64)
    # keep players off the room boundaries so the start sector is unambiguous
    for arr in (x_fixed, y_fixed):
        room_fixed = int(spec.room * FIXED_UNIT)
        rem = arr % room_fixed
        arr += np.where(rem < 20 * FIXED_UNIT, 20 * FIXED_UNIT - rem, 0)
        rem = arr % room_fixed
        arr -= np.where(rem > room_fixed - 20 * FIXED_UNIT, rem - (room_fixed - 20 * FIXED_UNIT), 0)
    bam = rng.integers(0, 1 << 32, size=n, dtype=np.int64)
    x = (x_fixed.astype(np.float32) / np.float32(FIXED_UNIT)).astype(np.float32)
    y = (y_fixed.astype(np.float32) / np.float32(FIXED_UNIT)).astype(np.float32)
    angle = (bam.astype(np.float32) * np.float32(gdstate.BAM_TO_RADIANS)).astype(np.float32)
    sector = gdscene.sector_at(sc, x, y)
    view_z = (sc.sector_heights[sector, 0] + np.float32(VIEW_HEIGHT)).astype(np.float32)

    lf[:, gdstate.L_X] = x
    lf[:, gdstate.L_Y] = y
    lf[:, gdstate.L_ANGLE] = angle
    lf[:, gdstate.L_VIEW_Z] = view_z
    lanes[:, gdstate.L_X_FIXED] = x_fixed
    lanes[:, gdstate.L_Y_FIXED] = y_fixed
    lanes[:, gdstate.L_ANGLE_BAM] = bam.astype(np.uint32).view(np.int32)
    lanes[:, gdstate.L_EPISODE_TIME] = rng.integers(1, 400, size=n)
    lanes[:, gdstate.L_BOB_FIXED] = rng.integers(0, 16 * FIXED_UNIT, size=n)
    lanes[:, gdstate.L_WEAPON] = rng.integers(0, 8, size=n)
    lanes[:, gdstate.L_WPN_COOLDOWN] = np.where(rng.random(n) < 0.5, 0, rng.integers(0, 20, size=n))
    lanes[:, gdstate.L_WPN_FIRE_COUNT] = rng.integers(0, 9, size=n)
    lanes[:, gdstate.L_WPN_READY_TICS] = rng.integers(0, 40, size=n)
    lanes[:, gdstate.L_WPN_RAISE] = np.where(rng.random(n) < 0.8, 0, rng.integers(0, 15, size=n))
    lanes[:, gdstate.L_WPN_LOWER] = rng.integers(0, 17, size=n)
    lanes[:, gdstate.L_WPN_PENDING] = np.where(rng.random(n) < 0.9, -1, rng.integers(0, 8, size=n))
    lf[:, gdstate.L_HEALTH] = rng.integers(0, 201, size=n).astype(np.float32)
    lf[:, gdstate.L_ARMOR] = rng.integers(0, 201, size=n).astype(np.float32)
    lf[:, gdstate.L_READY_AMMO] = rng.integers(0, 301, size=n).astype(np.float32)
    lf[:, gdstate.L_AMMO0:gdstate.L_AMMO3 + 1] = rng.integers(0, 301, size=(n, 4)).astype(np.float32)
    lanes[:, gdstate.L_WEAPONS_OWNED] = rng.integers(0, 64, size=n) | 3
    lanes[:, gdstate.L_FACE_INDEX] = rng.integers(0, 3, size=n)
    lanes[:, gdstate.L_PAIN_DIRECTION] = rng.integers(0, 3, size=n)
    lanes[:, gdstate.L_PAIN_TICS] = np.where(rng.random(n) < 0.8, 0, rng.integers(1, 35, size=n))
    lanes[:, gdstate.L_GRIN_TICS] = np.where(rng.random(n) < 0.9, 0, rng.integers(1, 71, size=n))
    lanes[:, gdstate.L_ATTACK_HELD] = np.where(rng.random(n) < 0.9, 0, rng.integers(70, 100, size=n))
    lanes[:, gdstate.L_FLAGS] = (rng.random(n) < 0.03).astype(np.int32) | ((rng.random(n) < 0.1).astype(np.int32) << 1)

    k = k_things
    kk = max(k if max_things is None else max_things, 1)
    things = np.zeros((n, kk, 4), dtype=np.int32)
    if k > 0:
        tx = rng.uniform(8.0, width - 8.0, size=(n, k)).astype(np.float32)
        ty = rng.uniform(8.0, height - 8.0, size=(n, k)).astype(np.float32)
        tsec = gdscene.sector_at(sc, tx.reshape(-1), ty.reshape(-1)).reshape(n, k)
        tz = sc.sector_heights[tsec, 0].astype(np.float32)
        sprite = rng.integers(0, len(sc.spr_atlas), size=(n, k)).astype(np.int64)
        alive = rng.random((n, k)) < 0.95
        bright = rng.random((n, k)) < 0.1
        style = rng.choice(np.asarray([-1, -1, -1, -1, 0, 1, -2]), size=(n, k)).astype(np.int64)
        things[:, :k, 0] = tx.view(np.int32)
        things[:, :k, 1] = ty.view(np.int32)
        things[:, :k, 2] = tz.view(np.int32)
        flags = alive.astype(np.int64) * gdstate.THING_ALIVE + bright.astype(np.int64) * gdstate.THING_BRIGHT
        word = (sprite & 0xFFFF) | (flags << 16) | ((style & 0xFF) << 24)
        things[:, :k, 3] = word.astype(np.uint32).view(np.int32)
    lanes[:, gdstate.L_THINGS] = k
    return lanes, things


def advance(sc: gdscene.Scene, lanes: np.ndarray, seed: int, turn_bam: int = 640 << 16, move: float = 6.0):
    """Turn every player a little and move it forward inside its room (numpy, in place)."""

    rng = np.random.default_rng(seed)
    spec = sc.meta["spec"]
    n = lanes.shape[0]
    lf = lanes.view(np.float32)
    bam = lanes[:, gdstate.L_ANGLE_BAM].view(np.uint32).astype(np.int64)
    bam = (bam + rng.integers(-2, 3, size=n) * turn_bam) & 0xFFFFFFFF
    ang = bam.astype(np.float64) * (2.0 * np.pi / (1 << 32))
    room_fixed = int(spec.room * FIXED_UNIT)
    for word, delta in ((gdstate.L_X_FIXED, np.cos(ang)), (gdstate.L_Y_FIXED, np.sin(ang))):
        cur = lanes[:, word].astype(np.int64)
        new = cur + np.round(delta * move * FIXED_UNIT).astype(np.int64)
        rem = new % room_fixed
        ok = (new // room_fixed == cur // room_fixed) & (rem > 20 * FIXED_UNIT) & (rem < room_fixed - 20 * FIXED_UNIT)
        lanes[:, word] = np.where(ok, new, cur)
    lanes[:, gdstate.L_ANGLE_BAM] = bam.astype(np.uint32).view(np.int32)
    lf[:, gdstate.L_X] = lanes[:, gdstate.L_X_FIXED].astype(np.float32) / np.float32(FIXED_UNIT)
    lf[:, gdstate.L_Y] = lanes[:, gdstate.L_Y_FIXED].astype(np.float32) / np.float32(FIXED_UNIT)
    lf[:, gdstate.L_ANGLE] = bam.astype(np.float32) * np.float32(gdstate.BAM_TO_RADIANS)
    lanes[:, gdstate.L_EPISODE_TIME] += 1
    return lanes
