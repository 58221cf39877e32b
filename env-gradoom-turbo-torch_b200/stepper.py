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
        jitter = rng.integers(0, 8 * FIXED_UNIT, size=n)   # no player exactly on the margin line
        rem = arr % room_fixed
        arr += np.where(rem < 20 * FIXED_UNIT, 20 * FIXED_UNIT - rem + jitter, 0)
        rem = arr % room_fixed
        arr -= np.where(rem > room_fixed - 20 * FIXED_UNIT, rem - (room_fixed - 20 * FIXED_UNIT) + jitter, 0)
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


def random_decals(sc: gdscene.Scene, lanes: np.ndarray, per_lane: int, slots: int, seed: int) -> np.ndarray:
    """Seeded bullet chips for every lane: ``(n, slots, 4) int32`` ``gd_decal`` rings.  Most chips sit
    where a ray through the lane's view meets the nearest line, on the viewer's side of it (what a
    hitscan impact leaves, src/gradoom/engine.py:6257-6340); a few are on the far side or on lines
    elsewhere.  Serials ascend in shuffled slot order; the other slots are free."""

    rng = np.random.default_rng(seed)
    n = lanes.shape[0]
    lf = lanes.view(np.float32)
    walls = sc.walls.astype(np.float64)
    sx, sy = walls[:, 0], walls[:, 1]
    ex, ey = walls[:, 2] - sx, walls[:, 3] - sy
    out = np.zeros((n, slots, 4), dtype=np.int32)
    out[:, :, 0] = -1
    of = out.view(np.float32)
    for lane in range(n):
        px, py, ang = float(lf[lane, gdstate.L_X]), float(lf[lane, gdstate.L_Y]), float(lf[lane, gdstate.L_ANGLE])
        where = rng.permutation(slots)[:per_lane]
        for i, slot in enumerate(where):
            if rng.random() < 0.85:
                a = ang + rng.uniform(-0.75, 0.75)
                rx, ry = np.cos(a), np.sin(a)
                den = rx * ey - ry * ex
                ok = np.abs(den) > 1e-9
                den = np.where(ok, den, 1.0)
                dist = ((sx - px) * ey - (sy - py) * ex) / den
                t = ((sx - px) * ry - (sy - py) * rx) / den
                dist = np.where(ok & (dist > 1e-3) & (t >= 0) & (t <= 1), dist, np.inf)
                w = int(np.argmin(dist))
                if not np.isfinite(dist[w]):
                    continue
                along = float(t[w])
            else:
                w, along = int(rng.integers(0, len(walls))), float(rng.random())
            side = int(ex[w] * (py - sy[w]) - ey[w] * (px - sx[w]) > 0)
            if rng.random() < 0.1:
                side = 1 - side
            style = int(rng.integers(0, 5)) + 5 * int(rng.integers(0, 2)) + 10 * int(rng.integers(0, 2)) + 20 * side
            out[lane, slot, 0] = 1000 + i
            out[lane, slot, 1] = (w & 0xFFFF) | (style << 16)
            of[lane, slot, 2] = np.float32(along)
            of[lane, slot, 3] = np.float32(rng.uniform(-8.0, 200.0))
    return out


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


class LaneStepper:
    """Device-resident state producer of the environment.

    The players move with the reference's own per-tic kinematics, computed by the CUDA
    library (``gd_player_tics``: keyboard turn ramp, thrust, wall slide, step-up, view-height
    easing, gravity; src/gradoom/engine.py:4344-4671, 3207-3498) on player records kept on the
    device.  Everything else is synthetic and makes no parity claim: reset places the
    players at seeded positions inside the rooms (the reference draws them from its own
    random streams), the things stand still, an ATTACK press kills one now and then (which
    feeds the per-lane statistics), episodes time out.  It exposes what ``GraDoomVecEnv``
    needs from a producer: ``reset``, ``step``, ``render_inputs``, ``signal_buffer``,
    ``pending_reset``, and ``bind_renderer`` (the kinematics kernel lives in the renderer's
    library; there is no fallback without it).
    """

    SIGNALS = 27  # width of the reference's signal buffer (src/gradoom/engine.py:509-539)

    def __init__(self, sc, num_envs, *, device, k_things=12, max_things=None, frame_skip=2,
                 episode_timeout=4200, seed=0):
        import torch

        self.torch = torch
        self.scene = sc
        self.spec = sc.meta["spec"]
        self.num_envs = num_envs
        self.device = torch.device(device)
        self.frame_skip = frame_skip
        self.episode_timeout = episode_timeout
        self.k = k_things
        self.max_things = k_things if max_things is None else max_things
        lanes, things = random_lanes(sc, num_envs, k_things, seed, max_things=self.max_things)
        self.lanes = torch.from_numpy(lanes).to(self.device)
        self.things = torch.from_numpy(things).to(self.device)
        self.floors = torch.as_tensor(sc.sector_heights[:, 0].astype(np.float32), device=self.device)
        self.signal_buffer = torch.zeros((num_envs, self.SIGNALS), dtype=torch.float32, device=self.device)
        self.pending_reset = torch.zeros(num_envs, dtype=torch.bool, device=self.device)
        self.lanes[:, gdstate.L_EPISODE_TIME] = 1
        self.ceilings = torch.as_tensor(sc.sector_heights[:, 1].astype(np.float32), device=self.device)
        self.players = torch.zeros((num_envs, gdstate.PLAYER_WORDS), dtype=torch.int32, device=self.device)
        self.button_weights = None
        self.renderer = None
        self._tick = 0
        self._players_from_lanes(torch.ones(num_envs, dtype=torch.bool, device=self.device))

    def bind_renderer(self, renderer):
        self.renderer = renderer

    def _players_from_lanes(self, mask):
        """Player records of freshly placed lanes: standing on the floor of their room."""

        torch = self.torch
        lanes, players = self.lanes, self.players
        room = float(self.spec.room)
        xf = lanes[:, gdstate.L_X_FIXED].to(torch.float32) / FIXED_UNIT
        yf = lanes[:, gdstate.L_Y_FIXED].to(torch.float32) / FIXED_UNIT
        col = torch.clamp((xf / room).to(torch.int64), 0, self.spec.cols - 1)
        row = torch.clamp((yf / room).to(torch.int64), 0, self.spec.rows - 1)
        sector = row * self.spec.cols + col
        floor, ceiling = self.floors[sector], self.ceilings[sector]
        fresh = torch.zeros_like(players)
        fresh[:, gdstate.P_X_FIXED] = lanes[:, gdstate.L_X_FIXED]
        fresh[:, gdstate.P_Y_FIXED] = lanes[:, gdstate.L_Y_FIXED]
        fresh[:, gdstate.P_ANGLE_BAM] = lanes[:, gdstate.L_ANGLE_BAM]
        for word, value in ((gdstate.P_Z, floor), (gdstate.P_VIEW_Z, floor + VIEW_HEIGHT),
                            (gdstate.P_VIEW_HEIGHT, torch.full_like(floor, VIEW_HEIGHT)), (gdstate.P_FLOOR_Z, floor),
                            (gdstate.P_CEILING_Z, ceiling), (gdstate.P_PREV_FLOOR_Z, floor)):
            fresh[:, word] = value.contiguous().view(torch.int32)
        fresh[:, gdstate.P_REACTION_TIME] = 7       # the input freeze after a spawn (src/gradoom/engine.py:81, 2407)
        fresh[:, gdstate.P_EPISODE_TIME] = lanes[:, gdstate.L_EPISODE_TIME]
        players.copy_(torch.where(mask[:, None], fresh, players))

    # deterministic per-lane pseudo random numbers in [0, 1)
    def _uniform(self, seeds, salt):
        torch = self.torch
        v = (seeds.to(torch.int64) * 2654435761 + salt * 40503 + 12345) & 0xFFFFFFFF
        v ^= v >> 15
        v = (v * 2246822519) & 0xFFFFFFFF
        v ^= v >> 13
        v = (v * 3266489917) & 0xFFFFFFFF
        v ^= v >> 16
        return v.to(torch.float64) / float(1 << 32)

    def _refresh_pose(self, x_fixed, y_fixed, bam, mask):
        torch = self.torch
        lanes = self.lanes
        room = float(self.spec.room)
        xf = x_fixed.to(torch.float32) / FIXED_UNIT
        yf = y_fixed.to(torch.float32) / FIXED_UNIT
        col = torch.clamp((xf / room).to(torch.int64), 0, self.spec.cols - 1)
        row = torch.clamp((yf / room).to(torch.int64), 0, self.spec.rows - 1)
        view_z = self.floors[row * self.spec.cols + col] + VIEW_HEIGHT
        angle = bam.to(torch.float32) * gdstate.BAM_TO_RADIANS
        signed_bam = torch.where(bam >= (1 << 31), bam - (1 << 32), bam)

        def put(word, value):
            lanes[:, word] = torch.where(mask, value.to(torch.int32), lanes[:, word])

        put(gdstate.L_X, xf.view(torch.int32))
        put(gdstate.L_Y, yf.view(torch.int32))
        put(gdstate.L_ANGLE, angle.view(torch.int32))
        put(gdstate.L_VIEW_Z, view_z.view(torch.int32))
        put(gdstate.L_X_FIXED, x_fixed)
        put(gdstate.L_Y_FIXED, y_fixed)
        put(gdstate.L_ANGLE_BAM, signed_bam)

    def reset(self, mask, seeds):
        torch = self.torch
        width = self.spec.cols * self.spec.room
        height = self.spec.rows * self.spec.room
        room_fixed = int(self.spec.room * FIXED_UNIT)
        margin = 20 * FIXED_UNIT

        def coordinate(extent, salt):
            v = (self._uniform(seeds, salt) * (extent - 48.0) + 24.0) * FIXED_UNIT
            v = v.to(torch.int64)
            jitter = (self._uniform(seeds, salt + 10) * (8 * FIXED_UNIT)).to(torch.int64)
            rem = v % room_fixed
            v = v + torch.where(rem < margin, margin - rem + jitter, torch.zeros_like(rem))
            rem = v % room_fixed
            return v - torch.where(rem > room_fixed - margin, rem - (room_fixed - margin) + jitter,
                                   torch.zeros_like(rem))

        x_fixed = coordinate(width, 1)
        y_fixed = coordinate(height, 2)
        bam = (self._uniform(seeds, 3) * float(1 << 32)).to(torch.int64) & 0xFFFFFFFF
        self._refresh_pose(x_fixed, y_fixed, bam, mask)
        self.lanes[:, gdstate.L_EPISODE_TIME] = torch.where(
            mask, torch.ones_like(self.lanes[:, gdstate.L_EPISODE_TIME]), self.lanes[:, gdstate.L_EPISODE_TIME])
        self.lanes[:, gdstate.L_FLAGS] = torch.where(mask, torch.zeros_like(self.lanes[:, 0]),
                                                     self.lanes[:, gdstate.L_FLAGS])
        if self.k > 0:
            word = self.things[:, :, 3]
            self.things[:, :, 3] = torch.where(mask[:, None], word | (THING_ALIVE_BIT), word)
        self.lanes[:, gdstate.L_BOB_FIXED] = torch.where(mask, torch.zeros_like(self.lanes[:, 0]),
                                                         self.lanes[:, gdstate.L_BOB_FIXED])
        self._players_from_lanes(mask)
        self.signal_buffer[mask] = 0
        self.signal_buffer[:, 1] = torch.where(mask, torch.full_like(self.signal_buffer[:, 1], 100.0),
                                               self.signal_buffer[:, 1])
        self.pending_reset &= ~mask

    def step(self, buttons):
        torch = self.torch
        lanes = self.lanes
        if self.renderer is None:
            raise RuntimeError("the lane stepper moves its players with the renderer's library: "
                               "bind_renderer() first (GraDoomVecEnv does it)")
        self._tick += 1
        b = buttons.to(torch.int64)
        if self.button_weights is None or self.button_weights.shape[0] != b.shape[1]:
            self.button_weights = 1 << torch.arange(b.shape[1], device=self.device, dtype=torch.int64)
        masks = (b * self.button_weights).sum(dim=1).to(torch.int32)
        # frame_skip game tics under the same buttons; the kernel also refreshes the pose words of the lane records
        self.renderer.player_tics(self.players, masks, self.frame_skip, self.episode_timeout, lanes=lanes)
        # an attack kills the first living thing once in a while
        rewards = torch.zeros(self.num_envs, dtype=torch.float32, device=self.device)
        if self.k > 0:
            lane_ids = torch.arange(self.num_envs, device=self.device, dtype=torch.int64)
            lucky = self._uniform(lane_ids + self._tick * 7919, 5) < 0.02
            victim = (self._uniform(lane_ids + self._tick * 104729, 6) * self.k).to(torch.int64).clamp(0, self.k - 1)
            word = self.things[lane_ids, victim, 3]
            alive = (word & THING_ALIVE_BIT) != 0
            kill = (b[:, 0] != 0) & lucky & alive
            self.things[lane_ids, victim, 3] = torch.where(kill, word & ~THING_ALIVE_BIT, word)
            rewards = kill.to(torch.float32)
        time = lanes[:, gdstate.L_EPISODE_TIME]
        truncated = time >= self.episode_timeout
        terminated = torch.zeros_like(truncated)
        self.pending_reset |= truncated
        sb = self.signal_buffer
        sb[:, 0] += rewards
        sb[:, 26] += rewards
        sb[:, 18] += rewards
        sb[:, 17] = time.to(torch.float32)
        sb[:, 20] = self.pending_reset.to(torch.float32)
        return rewards, terminated, truncated

    def render_inputs(self):
        return self.lanes, self.things


THING_ALIVE_BIT = gdstate.THING_ALIVE << 16
