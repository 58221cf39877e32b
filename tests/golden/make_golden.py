"""Generate the golden fixtures by running the upstream CPU renderer.

Run once on a machine that has the upstream sources:

    GRADOOM_REFERENCE_SRC=<upstream checkout>/src/gradoom python tests/golden/make_golden.py \
        [c1 c2 c3 c4 c1m stack flashes pitch fallback c2d c4d c1k state move_c1 move_c2 decals_c1 decals_c4 decals_c1m decals_fallback c1s c4s]

For each seeded synthetic scene it resets the upstream engine, injects K
monsters per lane, replays a seeded uniform action stream and, at a few
checkpoints, stores the renderer's inputs (lane and thing records built by this
package's packers from the engine state) together with the upstream outputs:
the 320x240 palette-indexed frame with status bar, the 84x84 observation of the
upstream float resize path, and the per-column ray tables.  The fixtures are
small ``.npz`` files next to this script; tests replay them without the
upstream sources.
"""

from __future__ import annotations

import dataclasses
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.environ.get("GRADOOM_GOLDEN_OUT", HERE)    # where the .npz files are written
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from __graft_entry__ import load_oracle, load_package  # noqa: E402

load_package()
oracle = load_oracle()
from gradoom_b200 import scene as gdscene, state as gdstate  # noqa: E402
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import ref_engine as refbridge  # noqa: E402

PLANS = {
    # name: (config, lanes, monsters per lane, checkpoints (agent steps))
    "c1": ("c1", 4, 4, (0, 12, 30)),
    "c2": ("c2", 2, 12, (0, 16)),
    "c3": ("c3", 2, 12, (0, 10)),
    "c4": ("c4", 1, 32, (0, 3)),
    "c1m": ("c1m", 4, 4, (0, 12, 30)),
    # deeper action streams on the two benchmark maps
    "c2d": ("c2", 8, 12, (0, 50, 150)),
    "c4d": ("c4", 4, 32, (0, 20, 60)),
    # lines split into projection fragments (engine.py:745-767, 11478-11545, 12310-12376)
    "c1s": ("c1s", 4, 4, (0, 12, 30)),
    "c4s": ("c4s", 4, 8, (0, 10, 25)),
}
# Plans whose skipped steps run with the upstream default (fast) observation renderer: the
# game dynamics never read a rendered frame, so the state at a checkpoint is the same
# (generate("c1") under both settings gives identical records).
FAST_STEPPING = {"c2d", "c4d"} | set(filter(None, os.environ.get("GRADOOM_GOLDEN_FAST", "").split(",")))
ACTION_SEED = 20260813


def action_matrix(act):
    am = torch.zeros((len(act.DEATHMATCH_ACTIONS), len(act.DEATHMATCH_BUTTONS)), dtype=torch.bool)
    for i, labels in enumerate(act.DEATHMATCH_ACTIONS):
        for label in labels:
            am[i, act.DEATHMATCH_BUTTONS.index(label)] = True
    return am


def make_engine(eng, scn, sc, n, k, seed, flashes=False):
    cs = refbridge.scene_to_compiled(sc, scn)
    e = eng.TorchDeathmatchEngine(cs, n, device=torch.device("cpu"), mask_hud=True,
                                  render_screen_flashes=flashes)
    e.render_frame = e.render_reference_frame
    e.reset(torch.ones(n, dtype=torch.bool), torch.arange(n) + 1)
    g = torch.Generator().manual_seed(seed)
    spec = sc.meta["spec"]
    e.enemy_x[:, :k] = torch.rand((n, k), generator=g) * (spec.cols * spec.room - 64) + 32
    e.enemy_y[:, :k] = torch.rand((n, k), generator=g) * (spec.rows * spec.room - 64) + 32
    sec = e._sector_at(e.enemy_x[:, :k].reshape(-1), e.enemy_y[:, :k].reshape(-1)).reshape(n, k)
    e.enemy_z[:, :k] = e.map.sector_heights[sec, 0]
    e.enemy_type[:, :k] = torch.randint(0, 6, (n, k), generator=g)
    e.enemy_alive[:, :k] = True
    e.enemy_angle[:, :k] = torch.rand((n, k), generator=g) * 6.28
    return e, g


def pack(e, blob, max_things=64):
    """The renderer's inputs for the engine's present state (CPU packer of the oracle)."""

    lanes, things, k = oracle.pack_state(blob, e, max_things)
    if k > max_things:
        raise ValueError(f"{k} drawable actors exceed the configured maximum of {max_things}")
    return lanes, things


def snapshot(e, blob, max_things):
    lanes, things = pack(e, blob, max_things)
    indexed = e._render_native_indexed_frame(include_hud=True).numpy()
    obs_float = e.render_reference_frame().numpy()
    return lanes, things, indexed, obs_float


def generate(name, eng, scn, act):
    cfg, n, k, checkpoints = PLANS[name]
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[cfg])
    e, g = make_engine(eng, scn, sc, n, k, seed=1234)
    blob = gdscene.pack_scene(sc)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED)
    max_things = 64
    out = {"config": np.asarray(cfg), "checkpoints": np.asarray(checkpoints)}
    offsets, coscorr = gdscene.ray_tables()
    out["ray_offsets"], out["ray_coscorr"] = offsets, coscorr
    step = 0
    if name in FAST_STEPPING:
        del e.render_frame          # back to the class default while stepping
    for ci, target in enumerate(checkpoints):
        while step < target:
            a = torch.randint(0, 17, (n,), generator=ag)
            _f, _r, term, trunc = e.step(am[a])
            done = term | trunc
            if bool(done.any()):
                e.reset(done, torch.arange(n) + 1000 * (step + 1))
            step += 1
        lanes, things, indexed, obs_float = snapshot(e, blob, max_things)
        used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
        out[f"lanes_{ci}"] = lanes
        out[f"things_{ci}"] = things[:, :used].copy()
        out[f"indexed_{ci}"] = indexed
        out[f"obs_float_{ci}"] = obs_float
        print(name, "checkpoint", target, "things", used, flush=True)
    np.savez_compressed(os.path.join(OUT, f"golden_{name}.npz"), **out)


def generate_stack(eng, scn, act):
    """Reset + four consecutive agent steps on c1: inputs of every render and the
    upstream four-frame stack after each of them (engine.py:9545-9548, 2443-2450)."""

    n, k = 2, 4
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1"])
    e, g = make_engine(eng, scn, sc, n, k, seed=77)
    blob = gdscene.pack_scene(sc)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED + 1)
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c1"), "ray_offsets": offsets, "ray_coscorr": coscorr}
    # a masked reset of lane 1 only, as the reference's auto-reset does
    mask = torch.tensor([False, True])
    e.reset(mask, torch.tensor([5, 6]))
    lanes, things = pack(e, blob)
    used = [max(int(lanes[:, gdstate.L_THINGS].max()), 1)]
    out["reset_mask"] = mask.numpy()
    out["lanes_reset"], out["things_reset"] = lanes, things
    out["frames_reset"] = e.frames.numpy().copy()
    for s in range(4):
        a = torch.randint(0, 17, (n,), generator=ag)
        e.step(am[a])
        lanes, things = pack(e, blob)
        used.append(max(int(lanes[:, gdstate.L_THINGS].max()), 1))
        out[f"lanes_{s}"], out[f"things_{s}"] = lanes, things
        out[f"frames_{s}"] = e.frames.numpy().copy()
    kmax = max(used)
    for key in list(out):
        if key.startswith("things_"):
            out[key] = out[key][:, :kmax].copy()
    np.savez_compressed(os.path.join(OUT, "golden_stack.npz"), **out)
    print("stack fixture done", flush=True)


def generate_fallback(eng, scn, act):
    """Poses that leave most of the view to the per-pixel flat fallback
    (engine.py:10956-11171) on the 64-sector map: a player exactly on a portal
    line, exactly on a vertex, 2**-15 beside a line, and on a line looking along it
    (standing in the doorway between two rooms).  The pose is written after the reset,
    public floats and retained fixed-point coordinates together."""

    n, k = 6, 12
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c2"])
    e, g = make_engine(eng, scn, sc, n, k, seed=97)
    blob = gdscene.pack_scene(sc)
    poses = [  # x, y, angle (degrees)
        (512.0, 600.0, 170.0),                # on the portal line x = 512, looking across it
        (768.0, 1024.0, 200.0),               # on the vertex shared by four rooms
        (1280.0 + 2.0 ** -15, 700.0, 95.0),   # two fixed-point steps beside a line
        (900.0, 1536.0, 0.0),                 # on the line y = 1536, looking along it
        (600.0, 512.0, 200.0),                # on a horizontal portal line
        (512.0, 600.0, 100.0),                # on the line x = 512, looking almost along it
    ]
    x = torch.tensor([p[0] for p in poses], dtype=torch.float32)
    y = torch.tensor([p[1] for p in poses], dtype=torch.float32)
    bam = torch.tensor([int(round(p[2] / 360.0 * (1 << 32))) & 0xFFFFFFFF for p in poses], dtype=torch.int64)
    e.x.copy_(x)
    e.y.copy_(y)
    e._x_fixed.copy_(torch.round(x.to(torch.float64) * 65536.0).to(torch.int64))
    e._y_fixed.copy_(torch.round(y.to(torch.float64) * 65536.0).to(torch.int64))
    e._angle_bam.copy_(bam)
    e.angle.copy_(bam.to(torch.float32) * gdstate.BAM_TO_RADIANS)
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c2"), "ray_offsets": offsets, "ray_coscorr": coscorr,
           "checkpoints": np.asarray([0])}
    lanes, things, indexed, obs_float = snapshot(e, blob, 64)
    used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
    out["lanes_0"], out["things_0"] = lanes, things[:, :used].copy()
    out["indexed_0"], out["obs_float_0"] = indexed, obs_float
    np.savez_compressed(os.path.join(OUT, "golden_fallback.npz"), **out)
    print("fallback fixture done", flush=True)


FALLBACK_POSES = [  # x, y, angle (degrees): see generate_fallback
    (512.0, 600.0, 170.0), (768.0, 1024.0, 200.0), (1280.0 + 2.0 ** -15, 700.0, 95.0),
    (900.0, 1536.0, 0.0), (600.0, 512.0, 200.0), (512.0, 600.0, 100.0),
]


def generate_decals(cfg, eng, scn, act, poses=None, name=None):
    """Bullet chips on the walls in view (engine.py:13747-13991): the scene carries decal bitmaps,
    the engine's decal rings are written directly (the way the upstream tests set state): per lane
    some forty chips where rays through the view meet the nearest line, at seeded heights, on the
    viewer's side of the line mostly, a few on the far side, a few on lines elsewhere, serials in
    shuffled slot order, free slots in between."""

    n, k = (4 if poses is None else len(poses)), 4
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[cfg])
    blob = gdscene.pack_scene(sc)
    e, g = make_engine(eng, scn, sc, n, k, seed=4242)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED + 11)
    del e.render_frame
    for step in range(12):
        _f, _r, term, trunc = e.step(am[torch.randint(0, 17, (n,), generator=ag)])
        done = term | trunc
        if bool(done.any()):
            e.reset(done, torch.arange(n) + 1000 * (step + 1))
    if poses is not None:          # stand on lines and vertices, as the fallback fixture does
        x = torch.tensor([p[0] for p in poses], dtype=torch.float32)
        y = torch.tensor([p[1] for p in poses], dtype=torch.float32)
        bam = torch.tensor([int(round(p[2] / 360.0 * (1 << 32))) & 0xFFFFFFFF for p in poses], dtype=torch.int64)
        e.x.copy_(x)
        e.y.copy_(y)
        e._x_fixed.copy_(torch.round(x.to(torch.float64) * 65536.0).to(torch.int64))
        e._y_fixed.copy_(torch.round(y.to(torch.float64) * 65536.0).to(torch.int64))
        e._angle_bam.copy_(bam)
        e.angle.copy_(bam.to(torch.float32) * gdstate.BAM_TO_RADIANS)
    rng = np.random.default_rng(99)
    walls = sc.walls.astype(np.float64)
    slots = e.hitscan_decal_serial.shape[1]
    serial = np.full((n, slots), -1, dtype=np.int32)
    wall = np.zeros((n, slots), dtype=np.int32)
    along = np.zeros((n, slots), dtype=np.float32)
    zs = np.zeros((n, slots), dtype=np.float32)
    style = np.zeros((n, slots), dtype=np.uint8)
    for lane in range(n):
        px, py, ang = float(e.x[lane]), float(e.y[lane]), float(e.angle[lane])
        chips = []
        for _ in range(44):
            if rng.random() < 0.85:
                a = ang + rng.uniform(-0.75, 0.75)
                rx, ry = np.cos(a), np.sin(a)
                sx, sy = walls[:, 0], walls[:, 1]
                ex, ey = walls[:, 2] - sx, walls[:, 3] - sy
                den = rx * ey - ry * ex
                ok = np.abs(den) > 1e-9
                den = np.where(ok, den, 1.0)
                dist = ((sx - px) * ey - (sy - py) * ex) / den
                t = ((sx - px) * ry - (sy - py) * rx) / den
                dist = np.where(ok & (dist > 1e-3) & (t >= 0) & (t <= 1), dist, np.inf)
                w = int(np.argmin(dist))
                if not np.isfinite(dist[w]):
                    continue
                tt = float(t[w])
            else:
                w, tt = int(rng.integers(0, len(walls))), float(rng.random())
            cross = (walls[w, 2] - walls[w, 0]) * (py - walls[w, 1]) - (walls[w, 3] - walls[w, 1]) * (px - walls[w, 0])
            side = int(cross > 0)
            if rng.random() < 0.1:
                side = 1 - side
            chips.append((w, tt, float(rng.uniform(-8.0, 200.0)), int(rng.integers(0, 5)) + 5 * int(rng.integers(0, 2))
                          + 10 * int(rng.integers(0, 2)) + 20 * side))
        where = rng.permutation(slots)[: len(chips)]
        for i, (slot, chip) in enumerate(zip(where, chips)):
            serial[lane, slot] = 1000 + i
            wall[lane, slot], along[lane, slot], zs[lane, slot], style[lane, slot] = chip
    e.hitscan_decal_serial.copy_(torch.from_numpy(serial))
    e.hitscan_decal_wall.copy_(torch.from_numpy(wall))
    e.hitscan_decal_along.copy_(torch.from_numpy(along))
    e.hitscan_decal_z.copy_(torch.from_numpy(zs))
    e.hitscan_decal_style.copy_(torch.from_numpy(style))
    e.hitscan_decal_count.copy_(torch.full((n,), 1000 + 44, dtype=torch.int64))
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray(cfg), "ray_offsets": offsets, "ray_coscorr": coscorr, "checkpoints": np.asarray([0]),
           "decal_serial": serial, "decal_wall": wall, "decal_along": along, "decal_z": zs, "decal_style": style}
    lanes, things, indexed, obs_float = snapshot(e, blob, 64)
    used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
    out["lanes_0"], out["things_0"] = lanes, things[:, :used].copy()
    out["indexed_0"], out["obs_float_0"] = indexed, obs_float
    # the same state with the rings emptied, to count what the chips changed
    e.hitscan_decal_serial.fill_(-1)
    bare = e._render_native_indexed_frame(include_hud=True).numpy()
    out["changed_pixels"] = np.asarray(int((bare != indexed).sum()))
    np.savez_compressed(os.path.join(OUT, f"golden_decals_{name or cfg}.npz"), **out)
    print("decal fixture", name or cfg, "done; pixels the chips changed:", int(out["changed_pixels"]), flush=True)



def generate_c1k(eng, scn, act):
    """The CPU configuration of the benchmark definition taken literally: c1, 4 lanes,
    uniform actions, a checkpoint after 1000 agent steps: the renderer's inputs, the
    indexed frame, and the four-frame stack (engine.py:9545-9548) together with the
    inputs of the four renders that filled it."""

    n, k, total = 4, 4, 1000
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1"])
    e, g = make_engine(eng, scn, sc, n, k, seed=1234)
    blob = gdscene.pack_scene(sc)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED)
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c1"), "ray_offsets": offsets, "ray_coscorr": coscorr,
           "checkpoints": np.asarray([total])}
    reference_frame = e.render_frame
    del e.render_frame              # fast default renderer while skipping (see FAST_STEPPING)
    resets = 0
    for step in range(total):
        if step == total - 8:
            e.render_frame = reference_frame
        a = torch.randint(0, 17, (n,), generator=ag)
        _f, _r, term, trunc = e.step(am[a])
        done = term | trunc
        if bool(done.any()):
            e.reset(done, torch.arange(n) + 1000 * (step + 1))
            resets += int(done.sum())
        if step >= total - 4:
            lanes, things = pack(e, blob)
            s = step - (total - 4)
            out[f"stack_lanes_{s}"], out[f"stack_things_{s}"] = lanes, things
            out[f"stack_done_{s}"] = done.numpy()
        if step % 100 == 0:
            print("c1k step", step, flush=True)
    lanes, things, indexed, obs_float = snapshot(e, blob, 64)
    used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
    kmax = max(used, *(int(out[f"stack_lanes_{s}"][:, gdstate.L_THINGS].max()) for s in range(4)))
    for s in range(4):
        out[f"stack_things_{s}"] = out[f"stack_things_{s}"][:, :kmax].copy()
    out["lanes_0"], out["things_0"] = lanes, things[:, :used].copy()
    out["indexed_0"], out["obs_float_0"] = indexed, obs_float
    out["frames"] = e.frames.numpy().copy()
    out["resets"] = np.asarray(resets)
    np.savez_compressed(os.path.join(OUT, "golden_c1k.npz"), **out)
    print("c1k fixture done; lane resets along the way:", resets, flush=True)


def generate_state(eng, scn, act):
    """The engine's own lane tensors with every actor class in use, and the frame the
    upstream renderer draws from them: c1 with twelve map items, 6 lanes, 40 agent steps
    of the uniform action stream, then effects written into a few slots of every class
    (the way the upstream tests set state).  Pins the state packer: tensors in, records
    out, frame equal."""

    n, k = 6, 4
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1i"])
    blob = gdscene.pack_scene(sc)
    e, g = make_engine(eng, scn, sc, n, k, seed=555)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED + 7)
    del e.render_frame
    for step in range(40):
        _f, _r, term, trunc = e.step(am[torch.randint(0, 17, (n,), generator=ag)])
        done = term | trunc
        if bool(done.any()):
            e.reset(done, torch.arange(n) + 1000 * (step + 1))
    spec = sc.meta["spec"]
    span_x, span_y = spec.cols * spec.room - 64, spec.rows * spec.room - 64

    def place(count):
        x = torch.rand((n, count), generator=g) * span_x + 32
        y = torch.rand((n, count), generator=g) * span_y + 32
        sec = e._sector_at(x.reshape(-1), y.reshape(-1)).reshape(n, count)
        return x, y, e.map.sector_heights[sec, 0] + 24.0

    lanes_with = lambda p: torch.rand((n, 1), generator=g) < p          # noqa: E731
    # corpses: slots 10..13, both death kinds, several stages
    e.enemy_x[:, 10:14], e.enemy_y[:, 10:14], z = place(4)
    e.enemy_z[:, 10:14] = z - 24.0
    e.enemy_death_type[:, 10:14] = torch.randint(0, 6, (n, 4), generator=g)
    e.enemy_death_extreme[:, 10:14] = torch.rand((n, 4), generator=g) < 0.4
    e.enemy_death_elapsed[:, 10:14] = torch.randint(0, 60, (n, 4), generator=g).to(torch.int32)
    e.enemy_death_tics[:, 10:14] = (torch.randint(0, 30, (n, 4), generator=g) * lanes_with(0.7)).to(torch.int32)
    # living monsters in every animation state
    e.enemy_attack_phase[:, :k] = torch.randint(0, 5, (n, k), generator=g).to(torch.int32)
    e.enemy_cooldown[:, :k] = torch.randint(0, 24, (n, k), generator=g).to(torch.int32)
    e.enemy_pain_tics[:, :k] = (torch.randint(0, 6, (n, k), generator=g) * (torch.rand((n, k), generator=g) < 0.3)).to(torch.int32)
    e.enemy_animation_tics[:, :k] = torch.randint(0, 200, (n, k), generator=g).to(torch.int32)
    e.enemy_target_slot[:, :k] = torch.randint(-2, 3, (n, k), generator=g)
    # player projectiles: flights in slots 0..2, impacts in slots 3..4
    e.projectile_x[:, 0:5], e.projectile_y[:, 0:5], e.projectile_z[:, 0:5] = place(5)
    e.projectile_velocity_x[:, 0:5] = torch.randn((n, 5), generator=g) * 10
    e.projectile_velocity_y[:, 0:5] = torch.randn((n, 5), generator=g) * 10
    e.projectile_type[:, 0:5] = torch.randint(0, 2, (n, 5), generator=g)
    e.projectile_age[:, 0:5] = torch.randint(0, 40, (n, 5), generator=g).to(torch.int32)
    e.projectile_alive[:, 0:3] = torch.rand((n, 3), generator=g) < 0.6
    e.projectile_impact_type[:, 3:5] = torch.randint(0, 3, (n, 2), generator=g)
    e.projectile_impact_tics[:, 3:5] = torch.randint(0, 16, (n, 2), generator=g).to(torch.int32)
    # enemy projectiles: flights 0..1, impacts 2..3
    e.enemy_projectile_x[:, 0:4], e.enemy_projectile_y[:, 0:4], e.enemy_projectile_z[:, 0:4] = place(4)
    e.enemy_projectile_velocity_x[:, 0:4] = torch.randn((n, 4), generator=g) * 10
    e.enemy_projectile_velocity_y[:, 0:4] = torch.randn((n, 4), generator=g) * 10
    e.enemy_projectile_age[:, 0:4] = torch.randint(0, 40, (n, 4), generator=g).to(torch.int32)
    e.enemy_projectile_alive[:, 0:2] = torch.rand((n, 2), generator=g) < 0.6
    e.enemy_projectile_impact_tics[:, 2:4] = torch.randint(0, 12, (n, 2), generator=g).to(torch.int32)
    # teleport fog, bullet puffs, dropped items
    e.teleport_fog_x[:, 5:8], e.teleport_fog_y[:, 5:8], e.teleport_fog_z[:, 5:8] = place(3)
    e.teleport_fog_tics[:, 5:8] = torch.randint(0, 73, (n, 3), generator=g).to(torch.int32)
    e.hitscan_puff_x[:, 0:4], e.hitscan_puff_y[:, 0:4], e.hitscan_puff_z[:, 0:4] = place(4)
    e.hitscan_puff_tics[:, 0:4] = torch.randint(0, 17, (n, 4), generator=g).to(torch.int32)
    e.drop_x[:, 20:23], e.drop_y[:, 20:23], z = place(3)
    e.drop_z[:, 20:23] = z - 24.0
    e.drop_type[:, 20:23] = torch.tensor([2007, 2002, 2001])[torch.randint(0, 3, (n, 3), generator=g)]
    e.drop_spawned[:, 20:23] = torch.rand((n, 3), generator=g) < 0.7
    # map items: some picked up, animation offsets spread
    e.item_available.copy_(torch.rand(e.item_available.shape, generator=g) < 0.8)
    e.item_animation_initial_tics.copy_(torch.randint(1, 7, e.item_animation_initial_tics.shape, generator=g).to(torch.int32))
    e.episode_time.copy_(torch.randint(1, 500, (n,), generator=g).to(torch.int32))
    e.player_dead[1] = True

    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c1i"), "ray_offsets": offsets, "ray_coscorr": coscorr,
           "checkpoints": np.asarray([0])}
    for _field, attr, _dtype, _shape in gdstate.ENGINE_STATE_POINTERS:
        out["state_" + attr] = getattr(e, attr).numpy().copy()
    lanes, things, indexed, obs_float = snapshot(e, blob, 64)
    used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
    out["lanes_0"], out["things_0"] = lanes, things[:, :used].copy()
    out["indexed_0"], out["obs_float_0"] = indexed, obs_float
    np.savez_compressed(os.path.join(OUT, "golden_state.npz"), **out)
    print("state fixture done; records per lane:", used, flush=True)


def generate_move(eng, scn, act, config):
    """Per-step player kinematics of the upstream engine (engine.py:4344-4671, 3207-3498):
    4 lanes, 300 agent steps of the uniform action stream with frame skip 2, monster spawning
    switched off so that nothing but the map and the voodoo doll acts on the player.  Stored:
    the player record after the reset and after every step, and the button masks."""

    n, steps = 4, 300
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS[config])
    e, g = make_engine(eng, scn, sc, n, 0, seed=31)
    del e.render_frame
    e.next_spawn_check.fill_(2_000_000_000)
    # two lanes start beside the outer walls, looking at them at a slant, so that the run
    # contains wall contacts, slides along both axes and corner stalls
    spec = sc.meta["spec"]
    size_x, size_y = spec.cols * spec.room, spec.rows * spec.room
    for lane, (x, y, degrees) in ((2, (40.0, float(round(size_y * 0.4)), 205.0)), (3, (size_x - 60.0, 36.0, 300.0))):
        sector = int(e._sector_at(torch.tensor([x]), torch.tensor([y]))[0])
        floor, ceiling = float(e.map.sector_heights[sector, 0]), float(e.map.sector_heights[sector, 1])
        bam = int(round(degrees / 360.0 * (1 << 32))) & 0xFFFFFFFF
        e._x_fixed[lane], e._y_fixed[lane] = int(x * 65536), int(y * 65536)
        e.x[lane], e.y[lane] = x, y
        e._angle_bam[lane] = bam
        e.angle[lane] = torch.tensor(bam, dtype=torch.int64).to(torch.float32) * gdstate.BAM_TO_RADIANS
        e.z[lane], e.view_z[lane] = floor, floor + 41.0
        e.player_floor_z[lane] = e.previous_player_floor_z[lane] = floor
        e.player_ceiling_z[lane] = ceiling
    am = action_matrix(act)
    weights = (1 << torch.arange(am.shape[1], dtype=torch.int64))
    ag = torch.Generator().manual_seed(ACTION_SEED + 11)
    out = {"config": np.asarray(config), "frame_skip": np.asarray(e.frame_skip),
           "episode_timeout": np.asarray(int(e.episode_timeout)),
           "players_reset": gdstate.player_records(e).numpy()}
    players, masks = [], []
    for step in range(steps):
        a = torch.randint(0, 17, (n,), generator=ag)
        # long runs of one action exercise the turn ramp and wall slides better than white noise
        if step % 40 >= 20:
            a = torch.full((n,), int(a[0]))
        buttons = am[a]
        _f, _r, term, trunc = e.step(buttons)
        assert not bool((term | trunc).any()), "the kinematics fixture expects no episode end"
        assert not bool(e.enemy_alive.any())
        assert torch.equal(e.x, e._x_fixed.to(torch.float32) / 65536) and torch.equal(e.y, e._y_fixed.to(torch.float32) / 65536)
        players.append(gdstate.player_records(e).numpy())
        masks.append((buttons.to(torch.int64) * weights).sum(dim=1).numpy().astype(np.uint32))
    out["players"] = np.stack(players)
    out["buttons"] = np.stack(masks)
    np.savez_compressed(os.path.join(OUT, f"golden_move_{config}.npz"), **out)
    print("move fixture done:", config, flush=True)


def generate_pitch(eng, scn, act):
    """c1 with the view pitched up and down (engine.py:9622-9631 and every use of the
    pitched view centre): inputs, indexed frames and observations."""

    n, k = 4, 4
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1"])
    e, g = make_engine(eng, scn, sc, n, k, seed=2468)
    blob = gdscene.pack_scene(sc)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED + 3)
    for _ in range(9):
        e.step(am[torch.randint(0, 17, (n,), generator=ag)])
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c1"), "ray_offsets": offsets, "ray_coscorr": coscorr,
           "checkpoints": np.asarray([0, 1, 2])}
    # BAM pitches: +-4, +-11, +-20, +-28 degrees and two odd values
    degrees = [(4.0, -4.0, 11.0, -11.0), (20.0, -20.0, 28.0, -28.0), (0.37, -7.77, 15.5, -1.0)]
    for ci, row in enumerate(degrees):
        bam = torch.tensor([int(round(d / 360.0 * (1 << 32))) for d in row], dtype=torch.int64)
        e._pitch_bam.copy_(bam)
        e.pitch.copy_(bam.to(torch.float32) * (2.0 * np.pi / (1 << 32)))
        lanes, things, indexed, obs_float = snapshot(e, blob, 64)
        used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
        out[f"lanes_{ci}"] = lanes
        out[f"things_{ci}"] = things[:, :used].copy()
        out[f"indexed_{ci}"] = indexed
        out[f"obs_float_{ci}"] = obs_float
    np.savez_compressed(os.path.join(OUT, "golden_pitch.npz"), **out)
    print("pitch fixture done", flush=True)


def generate_flashes(eng, scn, act):
    """c1 with the damage / bonus screen blends switched on (engine.py:15385-15397):
    inputs, the blended RGB24 frame and the observation derived from it."""

    n, k = 4, 4
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1"])
    e, g = make_engine(eng, scn, sc, n, k, seed=4321, flashes=True)
    blob = gdscene.pack_scene(sc)
    am = action_matrix(act)
    ag = torch.Generator().manual_seed(ACTION_SEED + 2)
    for _ in range(6):
        e.step(am[torch.randint(0, 17, (n,), generator=ag)])
    offsets, coscorr = gdscene.ray_tables()
    out = {"config": np.asarray("c1"), "ray_offsets": offsets, "ray_coscorr": coscorr,
           "damage_alpha": e._damage_to_alpha.numpy().astype(np.float32)}
    cases = [((0, 0, 0, 0), (0, 0, 0, 0)), ((7, 40, 100, 113), (0, 3, 6, 20)), ((1, 0, 63, 30), (16, 1, 0, 9))]
    for ci, (damage, bonus) in enumerate(cases):
        e.damage_count.copy_(torch.tensor(damage, dtype=torch.int32))
        e.bonus_count.copy_(torch.tensor(bonus, dtype=torch.int32))
        lanes, things = pack(e, blob)
        used = max(int(lanes[:, gdstate.L_THINGS].max()), 1)
        out[f"lanes_{ci}"] = lanes
        out[f"things_{ci}"] = things[:, :used].copy()
        out[f"rgb_{ci}"] = e.render_native_frame(include_hud=True).numpy()
        out[f"obs_float_{ci}"] = e.render_reference_frame().numpy()
    np.savez_compressed(os.path.join(OUT, "golden_flashes.npz"), **out)
    print("flash fixture done", flush=True)


def main(argv):
    eng, scn, act = refbridge.load_reference()
    names = argv or ["c1", "c2", "c3", "c4", "c1m", "stack", "flashes", "pitch"]
    for name in names:
        if name == "stack":
            generate_stack(eng, scn, act)
        elif name == "flashes":
            generate_flashes(eng, scn, act)
        elif name == "pitch":
            generate_pitch(eng, scn, act)
        elif name in ("move_c1", "move_c2"):
            generate_move(eng, scn, act, name[len("move_"):])
        elif name == "state":
            generate_state(eng, scn, act)
        elif name == "fallback":
            generate_fallback(eng, scn, act)
        elif name == "c1k":
            generate_c1k(eng, scn, act)
        elif name in ("decals_c1", "decals_c4", "decals_c1m"):
            generate_decals({"decals_c1": "c1d", "decals_c4": "c4d", "decals_c1m": "c1md"}[name], eng, scn, act)
        elif name == "decals_fallback":
            generate_decals("c2dec", eng, scn, act, poses=FALLBACK_POSES, name="fallback")
        else:
            generate(name, eng, scn, act)


if __name__ == "__main__":
    main(sys.argv[1:])
