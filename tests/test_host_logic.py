"""Host-side logic that needs no GPU: blob packing, state packing, the C ABI's
export table, the boundary's validation errors and the lane-sharding helpers."""

import ctypes
import os
import re
import types

import numpy as np
import pytest
import torch

import __graft_entry__ as entry

ROOT = entry.ROOT


def test_blob_header_and_sections_are_consistent(pkg, scenes):
    from gradoom_b200 import scene as gdscene

    sc, blob = scenes("c1")
    header = blob[: gdscene.GD_HDR_WORDS * 4].view(np.int32)
    assert header[gdscene.H["MAGIC"]] == gdscene.GD_MAGIC
    assert header[gdscene.H["BYTES"]] == blob.size
    assert header[gdscene.H["WALLS"]] == sc.num_walls == 40
    assert header[gdscene.H["SECTORS"]] == 16
    assert header[gdscene.H["UNSUPPORTED"]] == 0
    offsets = header[gdscene.GD_HDR_SECTION0: gdscene.GD_HDR_SECTION0 + len(gdscene.SEC)]
    assert (offsets % 16 == 0).all() and (np.diff(offsets) > 0).all() and offsets[-1] < blob.size
    # the layout header and the packer agree on the section list
    text = open(os.path.join(ROOT, "include", "gradoom_b200_layout.h")).read()
    declared = re.findall(r"^\s+GD_S_([A-Z0-9_]+)", text, flags=re.M)
    declared = [d for d in declared if d != "COUNT"]
    assert declared == list(gdscene._SECTIONS)
    version = int(re.search(r"#define GD_VERSION (\d+)", text).group(1))
    assert version == gdscene.GD_VERSION


def test_fine_tables_have_the_doom_landmarks(pkg):
    from gradoom_b200 import scene as gdscene

    sine = gdscene.fine_sine_table()
    assert sine[0] == 0 and sine[2048] == 65536 and sine[6144] == -65536 and sine[4096] == 0
    assert sine[1] == 50 and sine[1024] == 46340
    tan = gdscene.fine_tangent_table()
    assert len(tan) == 4096 and tan[2048] == 0 and tan[3072] == 65536


def test_generator_orientation_front_sector_on_the_right(pkg, scenes):
    sc, _ = scenes("c2")
    for w in range(sc.num_walls):
        x1, y1, x2, y2 = sc.walls[w]
        front = sc.wall_sectors[w, 0]
        r, c = divmod(int(front), 8)
        cx, cy = (c + 0.5) * 256.0, (r + 0.5) * 256.0
        cross = (x2 - x1) * (cy - y1) - (y2 - y1) * (cx - x1)
        assert cross < 0  # room centre on the right of v1 -> v2


def test_state_packer_lane_fields(pkg, oracle, scenes):
    """Lane records from engine-shaped tensors (src/gradoom/engine.py:1658-1739, 2122-2133,
    4673-4676, 10648-10658), through the CPU packer that checks the library's kernel."""

    from conftest import fake_engine
    from gradoom_b200 import state as gdstate

    _sc, blob = scenes("c1")
    e = fake_engine(3, seed=5)
    e.player_dead = torch.tensor([False, True, False])
    e.mugshot_ouch = torch.tensor([True, False, False])
    e.selected_weapon = torch.tensor([1, 3, 6])
    e.selected_weapon_variant = torch.tensor([True, True, False])
    e.weapons = torch.tensor([[1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 1], [1, 0, 0, 0, 0, 0]], dtype=torch.float32)
    lanes, things, k = oracle.pack_state(blob, e, 64)
    assert lanes.shape == (3, 32) and lanes.dtype == np.int32 and things.shape == (3, 64, 4)
    assert np.array_equal(lanes[:, gdstate.L_X].view(np.float32), e.x.numpy())
    assert np.array_equal(lanes[:, gdstate.L_X_FIXED], e._x_fixed.numpy())
    assert np.array_equal(lanes[:, gdstate.L_ANGLE_BAM].view(np.uint32), e._angle_bam.numpy().astype(np.uint32))
    assert lanes[:, gdstate.L_FLAGS].tolist() == [2, 1, 0]
    assert lanes[:, gdstate.L_THINGS].tolist() == [k, k, k] and 0 < k <= 64
    # slot 1 + variant -> chainsaw (1); slot 3 + variant -> super shotgun (4); slot 6 -> plasma (7)
    assert lanes[:, gdstate.L_WEAPON].tolist() == [1, 4, 7]
    assert lanes[:, gdstate.L_WEAPONS_OWNED].tolist() == [3, 0b100111, 1]
    # an overridden public coordinate wins over the retained fixed value
    e.x = e.x + 1.0
    lanes2, _, _ = oracle.pack_state(blob, e, 64)
    assert np.array_equal(lanes2[:, gdstate.L_X_FIXED], np.round(e.x.numpy() * 65536).astype(np.int32))
    # screen flashes travel in the flag word only when asked for
    e.damage_count = torch.tensor([7, 200, 0], dtype=torch.int32)
    e.bonus_count = torch.tensor([1, 2, 300], dtype=torch.int32)
    lanes3, _, _ = oracle.pack_state(blob, e, 64, render_screen_flashes=True)
    assert ((lanes3[:, gdstate.L_FLAGS] >> 8) & 0xFF).tolist() == [7, 113, 0]
    assert ((lanes3[:, gdstate.L_FLAGS] >> 16) & 0xFF).tolist() == [1, 2, 255]
    assert (lanes3[:, gdstate.L_FLAGS] & 4).tolist() == [4, 4, 4]


def test_sprite_rotation_known_answers(pkg, oracle, scenes):
    """Upstream tests/test_rendering.py:31-52: a viewer east / north / west / south of an
    actor that faces east sees rotations 0, 2, 4, 6; just below the -pi/8 boundary is 0."""

    import math

    from conftest import fake_engine

    sc, blob = scenes("c1")
    e = fake_engine(5, seed=9)
    for name in ("enemy_alive", "enemy_death_tics", "teleport_fog_tics", "drop_spawned", "projectile_alive",
                 "projectile_impact_tics", "enemy_projectile_alive", "enemy_projectile_impact_tics",
                 "hitscan_puff_tics", "enemy_pain_tics", "enemy_attack_phase", "enemy_animation_tics"):
        getattr(e, name).zero_()
    e.enemy_alive[:, 0] = True
    e.enemy_type[:, 0] = 4
    e.enemy_target_slot[:, 0] = -1
    e.enemy_x[:, 0], e.enemy_y[:, 0], e.enemy_angle[:, 0] = 500.0, 500.0, 0.0
    boundary = torch.tensor(-math.pi / 8, dtype=torch.float32)
    below = torch.nextafter(boundary, torch.tensor(float("-inf")))
    viewer = torch.tensor((0.0, math.pi / 2, math.pi, -math.pi / 2, float(below)))
    e.x = 500.0 + 100.0 * torch.cos(viewer)
    e.y = 500.0 + 100.0 * torch.sin(viewer)
    e._x_fixed = torch.round(e.x * 65536).to(torch.int64)
    e._y_fixed = torch.round(e.y * 65536).to(torch.int64)
    _lanes, things, k = oracle.pack_state(blob, e, 8)
    sprites = things[:, 0, 3] & 0xFFFF
    assert k == 1 + (len(sc.player_starts) - 1)
    assert sprites[:4].tolist() == [int(sc.enemy_walk_ids[4, 0, r]) for r in (0, 2, 4, 6)]
    assert sprites[4] in (int(sc.enemy_walk_ids[4, 0, 0]), int(sc.enemy_walk_ids[4, 0, 7]))


def test_engine_state_struct_matches_the_header(pkg):
    """The ctypes mirror lists the fields of ``struct gd_engine_state`` in the header's order."""

    from gradoom_b200 import state as gdstate

    text = open(os.path.join(entry.ROOT, "include", "gradoom_b200.h")).read()
    body = text[text.index("typedef struct gd_engine_state {"):text.index("} gd_engine_state;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        tail = re.sub(r"^(const\s+)?\w+\s+", "", decl)
        names += [part.strip().lstrip("*").strip() for part in tail.split(",")]
    mirror = [name for name, _ in gdstate.EngineStateStruct._fields_]
    assert names == mirror


def test_scene_from_the_reference_scenario_container(pkg, scenes):
    """A ``CompiledScenario``-shaped object (src/gradoom/scenario.py:302-410) converts into the
    same blob as the Scene it was made from; one without the native assets is refused."""

    import sys

    sys.path.insert(0, os.path.join(entry.ROOT, "oracle"))
    import ref_engine
    from gradoom_b200 import scene as gdscene

    sc, blob = scenes("c1i")
    container = ref_engine.scene_to_compiled(sc, types.SimpleNamespace(CompiledScenario=types.SimpleNamespace))
    back = gdscene.from_compiled_scenario(container)
    assert np.array_equal(gdscene.pack_scene(back), blob)
    # one fragment per line (what the upstream compiler writes for any map but its pinned one) changes
    # nothing; a line the node builder split arrives as projection fragments in the blob
    W = len(sc.walls)
    container.wall_projection_fragments_fixed = np.zeros((W, 2, 4), dtype=np.int64)
    container.wall_projection_fragment_mask = np.zeros((W, 2), dtype=bool)
    container.wall_projection_fragment_mask[:, 0] = True
    assert np.array_equal(gdscene.pack_scene(gdscene.from_compiled_scenario(container)), blob)
    container.wall_projection_fragment_mask[3, 1] = True
    container.wall_projection_fragments_fixed[3] = ((0, 0, 65536, 0), (65536, 0, 131072, 3))
    split = gdscene.pack_scene(gdscene.from_compiled_scenario(container))
    header = split[: gdscene.GD_HDR_WORDS * 4].view(np.int32)
    assert header[gdscene.H["FRAGMENTS"]] == 2
    off = split[header[gdscene.GD_HDR_SECTION0 + gdscene.SEC["FRAG_OFF"]]:].view(np.int32)[: W + 1]
    assert off[3] == 0 and off[4] == 2 and off[-1] == 2
    fixed = split[header[gdscene.GD_HDR_SECTION0 + gdscene.SEC["FRAG_FIXED"]]:].view(np.int32)[:8]
    assert fixed.tolist() == [0, 0, 65536, 0, 65536, 0, 131072, 3]
    container.wall_projection_fragment_mask = None
    with pytest.raises(ValueError):
        gdscene.from_compiled_scenario(container)
    container.wall_projection_fragments_fixed = None
    container.texture_index_atlas = None
    with pytest.raises(ValueError):
        gdscene.from_compiled_scenario(container)


def test_pack_things_roundtrip(pkg):
    from gradoom_b200 import state as gdstate

    x = torch.tensor([[1.5, -2.0]]); y = torch.tensor([[3.0, 4.0]]); z = torch.tensor([[0.0, 8.0]])
    things = gdstate.pack_things(x, y, z, torch.tensor([[7, 300]]), torch.tensor([[True, False]]),
                                 torch.tensor([[False, True]]), torch.tensor([[-2, 1]]), pad_to=4).numpy()
    assert things.shape == (1, 4, 4)
    assert things[0, 0, 0].view(np.float32) == np.float32(1.5)
    word = things[0, :2, 3].view(np.uint32)
    assert (word & 0xFFFF).tolist() == [7, 300]
    assert ((word >> 16) & 0xFF).tolist() == [1, 2]
    assert (word >> 24).astype(np.uint8).view(np.int8).tolist() == [-2, 1]


def test_library_exports_every_declared_symbol(pkg):
    from gradoom_b200 import native

    header = open(os.path.join(ROOT, "include", "gradoom_b200.h")).read()
    declared = set(re.findall(r"\b(gd_[a-z_]+)\s*\(", header))
    assert declared == set(native.EXPORTS)
    if not os.path.exists(native.LIBRARY):
        entry.build()
    lib = ctypes.CDLL(native.LIBRARY)
    for name in declared:
        assert getattr(lib, name) is not None
    lib.gd_error_string.restype = ctypes.c_char_p
    assert lib.gd_error_string(0) == b"ok"
    assert b"scratch" in lib.gd_error_string(-7)


def test_renderer_refuses_cpu_devices(pkg, scenes):
    from gradoom_b200 import native

    _sc, blob = scenes("c1")
    with pytest.raises(native.NativeError):
        native.Renderer(blob, "cpu", 4)


def test_boundary_validation_raises_the_reference_exception_types(pkg):
    from gradoom_b200 import env

    dev = torch.device("cpu")
    ok = torch.zeros(4, dtype=torch.int64)
    assert env.require_device_tensor(ok, "actions", device=dev, shape=(4,), dtypes=(torch.int64,)) is ok
    with pytest.raises(TypeError):
        env.require_device_tensor([0, 1, 2, 3], "actions", device=dev, shape=(4,), dtypes=(torch.int64,))
    with pytest.raises(ValueError):
        env.require_device_tensor(torch.zeros(3, dtype=torch.int64), "actions", device=dev, shape=(4,),
                                  dtypes=(torch.int64,))
    with pytest.raises(TypeError):
        env.require_device_tensor(torch.zeros(4), "actions", device=dev, shape=(4,), dtypes=(torch.int64,))
    with pytest.raises(TypeError):
        env.check_lane_index(True, 4)      # upstream tests/test_turbo_api_contract.py:509-519
    with pytest.raises(IndexError):
        env.check_lane_index(4, 4)
    assert env.check_lane_index(np.int64(2), 4) == 2
    m = env.action_matrix(dev)
    assert m.shape == (17, 20) and m[0].sum() == 0 and m[8].tolist().count(True) == 2


def test_lane_slices_partition_the_global_lanes(pkg):
    from gradoom_b200 import stats

    lanes = [i for r in range(8) for i in stats.lane_slice(r, 8, 8192)]
    assert lanes == list(range(65536))
    with pytest.raises(ValueError):
        stats.lane_slice(8, 8, 4)
    sb = torch.arange(3 * 27, dtype=torch.float32).reshape(3, 27)
    block = stats.local_stats(sb)
    assert block.shape == (3, 4) and block[1].tolist() == [27.0, 44.0, 45.0, 53.0]
    assert torch.equal(stats.gather_lane_stats(sb), block)


def test_random_lanes_are_valid_and_deterministic(pkg, scenes):
    from gradoom_b200 import stepper, state as gdstate

    sc, _ = scenes("c2")
    a = stepper.random_lanes(sc, 16, 12, seed=3)
    b = stepper.random_lanes(sc, 16, 12, seed=3)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    lanes = a[0]
    x = lanes[:, gdstate.L_X].view(np.float32)
    assert ((x > 0) & (x < 2048)).all()
    assert (lanes[:, gdstate.L_THINGS] == 12).all()


def test_decal_records_follow_the_record_layout(pkg, oracle):
    """gd_decal (include/gradoom_b200_layout.h): serial, wall | style << 16, along, z in 16 bytes; the
    torch packer, the test helper and the oracle's record type agree."""

    import types

    import torch

    from conftest import decal_rings
    from gradoom_b200 import state as gdstate

    rng = np.random.default_rng(3)
    data = {"decal_serial": rng.integers(-1, 500, size=(3, 16)).astype(np.int32),
            "decal_wall": rng.integers(0, 800, size=(3, 16)).astype(np.int32),
            "decal_style": rng.integers(0, 40, size=(3, 16)).astype(np.uint8),
            "decal_along": rng.random((3, 16)).astype(np.float32),
            "decal_z": rng.uniform(-8, 200, size=(3, 16)).astype(np.float32)}
    src = types.SimpleNamespace(**{f"hitscan_{k}": torch.from_numpy(v) for k, v in data.items()})
    rec = gdstate.decal_records(src).numpy()
    assert np.array_equal(rec, decal_rings(data))
    assert oracle.DECAL_DTYPE.itemsize == 16
    typed = rec.view(oracle.DECAL_DTYPE)[..., 0]
    assert np.array_equal(typed["serial"], data["decal_serial"]) and np.array_equal(typed["wall"], data["decal_wall"])
    assert np.array_equal(typed["style"], data["decal_style"]) and np.array_equal(typed["z"], data["decal_z"])
    again = torch.zeros((3, 16, 4), dtype=torch.int32)
    assert gdstate.decal_records(src, out=again) is again and np.array_equal(again.numpy(), rec)


def test_wall_fine_angles_of_axis_aligned_and_diagonal_lines(pkg):
    from gradoom_b200 import scene as gdscene

    walls = np.asarray([[0, 0, 64, 0], [0, 0, 0, 64], [64, 0, 0, 0], [0, 64, 0, 0], [0, 0, 64, 64], [64, 64, 0, 0],
                        [0, 64, 64, 0]], dtype=np.float32)
    fine = gdscene.wall_fine_angles(walls)
    assert fine[:, 0].tolist() == [0, 2048, 4096, 6144, 1024, 5120, 7168]
    assert fine[:, 1].tolist() == [4096, 6144, 0, 2048, 5120, 1024, 3072]
