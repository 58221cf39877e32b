"""Parity of the CUDA path, called through the C ABI, with the CPU oracle and
with the fixtures recorded from the upstream renderer.

Bar: palette-indexed frames, RGB frames, observations and frame stacks equal
the oracle bit for bit; against the upstream's float32 resize the observation
is within 1 LSB (upstream tests/test_rendering.py:112-139 grants the same).
"""

import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import engine_from_fixture, fake_engine, load_golden, pad_things

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _renderer(blob, k):
    from gradoom_b200 import native

    return native.Renderer(blob, DEV, k)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c1m", "pitch", "fallback", "c2d", "c4d", "c1k", "c1s", "c4s"])
def test_cuda_matches_upstream_fixtures(name, pkg, oracle, scenes):
    data = load_golden(name)
    _sc, blob = scenes(str(data["config"]), (data["ray_offsets"], data["ray_coscorr"]))
    r = _renderer(blob, 64)
    for ci in range(len(data["checkpoints"])):
        lanes, things = data[f"lanes_{ci}"], pad_things(data[f"things_{ci}"], 64)
        obs, indexed, rgb = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True, rgb=True)
        r.check_status()
        assert np.array_equal(indexed.cpu().numpy(), data[f"indexed_{ci}"])
        assert np.array_equal(rgb.cpu().numpy(), oracle.rgb(blob, data[f"indexed_{ci}"]))
        expected = oracle.render(blob, lanes, things)["obs"]
        assert np.array_equal(obs.cpu().numpy(), expected)
        diff = np.abs(obs.cpu().numpy().astype(int) - data[f"obs_float_{ci}"].astype(int))
        assert diff.max() <= 1


@pytest.mark.parametrize("name,n,k,seed", [("c1", 64, 4, 1), ("c2", 96, 12, 2), ("c3", 48, 12, 3),
                                           ("c4", 12, 32, 4), ("c2", 1, 0, 5), ("c1", 3, 1, 6),
                                           ("c1m", 48, 4, 7), ("c1s", 64, 4, 8), ("c4s", 48, 8, 9)])
def test_cuda_matches_oracle_on_seeded_lanes(name, n, k, seed, pkg, oracle, scenes):
    from gradoom_b200 import stepper

    sc, blob = scenes(name)
    lanes, things = stepper.random_lanes(sc, n, k, seed=seed)
    expected = oracle.render(blob, lanes, things, mask_hud=True)
    r = _renderer(blob, k)
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])


def test_views_pitched_to_the_ends_of_the_tangent_table_match_the_oracle(pkg, oracle, scenes):
    """Pitch values that index the first and last entries of the fine-tangent table put the screen centre
    tens of thousands of rows off screen: the visplane pixels then take the 64-bit form of their light
    term (the 32-bit form serves every pitch short of +-89.5 degrees), and everything else must hold too."""

    from gradoom_b200 import state as gdstate, stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 12, 4, seed=21)
    for lane, index in enumerate([0, 1, 2, 3, 8, 40, 4095, 4094, 4093, 4088, 4050, 2048]):
        lanes[lane, gdstate.L_PITCH_BAM] = 0x40000000 - (index << 19)
    expected = oracle.render(blob, lanes, things, mask_hud=True)
    r = _renderer(blob, 4)
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])
    only, _, _ = r.frames(_dev(lanes), _dev(things), obs=True)          # the observation-only configuration
    assert np.array_equal(only.cpu().numpy(), expected["obs"])


def test_unmasked_observation_includes_the_status_bar(pkg, oracle, scenes):
    from gradoom_b200 import stepper

    sc, blob = scenes("c3")
    lanes, things = stepper.random_lanes(sc, 8, 6, seed=9)
    expected = oracle.render(blob, lanes, things, mask_hud=False)
    r = _renderer(blob, 6)
    obs, _, _ = r.frames(_dev(lanes), _dev(things), obs=True, mask_hud=False)
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])
    masked, _, _ = r.frames(_dev(lanes), _dev(things), obs=True, mask_hud=True)
    assert not np.array_equal(masked.cpu().numpy()[:, 74:], obs.cpu().numpy()[:, 74:])
    assert masked.cpu().numpy()[:, 75:].max() == 0


def test_frames_without_status_bar_have_black_rows(pkg, scenes):
    from gradoom_b200 import stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 4, 4, seed=2)
    r = _renderer(blob, 4)
    _, a, _ = r.frames(_dev(lanes), _dev(things), indexed=True, include_hud=False)
    _, b, _ = r.frames(_dev(lanes), _dev(things), indexed=True, include_hud=True)
    assert a[:, 208:].max().item() == 0
    assert torch.equal(a[:, :208], b[:, :208]) and b[:, 208:].max().item() > 0


def test_stack_roll_and_masked_reset_fill(pkg, oracle, scenes):
    """engine.py:9545-9548 (roll + append) and 2443-2450 (masked fill)."""

    from gradoom_b200 import stepper

    sc, blob = scenes("c1")
    n, k = 16, 4
    r = _renderer(blob, k)
    rng = np.random.default_rng(0)
    stack_ref = rng.integers(0, 256, size=(n, 4, 84, 84), dtype=np.uint8)
    stack = _dev(stack_ref)
    lanes, things = stepper.random_lanes(sc, n, k, seed=21)
    mask = rng.random(n) < 0.5
    mask[0], mask[1] = True, False
    obs = oracle.render(blob, lanes, things)["obs"]
    oracle.stack_update(stack_ref, obs, reset_mask=mask)
    r.reset(_dev(lanes), _dev(things), _dev(mask), stack)
    assert np.array_equal(stack.cpu().numpy(), stack_ref)
    for step in range(5):
        stepper.advance(sc, lanes, seed=100 + step)
        obs = oracle.render(blob, lanes, things)["obs"]
        oracle.stack_update(stack_ref, obs)
        r.step(_dev(lanes), _dev(things), stack)
        assert np.array_equal(stack.cpu().numpy(), stack_ref), f"step {step}"
    r.check_status()


def test_cuda_replays_the_upstream_stack_fixture(pkg, oracle, scenes):
    data = load_golden("stack")
    _sc, blob = scenes("c1", (data["ray_offsets"], data["ray_coscorr"]))
    r = _renderer(blob, 64)
    stack = _dev(data["frames_reset"])
    r.reset(_dev(data["lanes_reset"]), _dev(pad_things(data["things_reset"], 64)), _dev(data["reset_mask"]), stack)
    masked = data["reset_mask"].astype(bool)
    got = stack.cpu().numpy()
    assert np.array_equal(got[~masked], data["frames_reset"][~masked])
    assert np.abs(got[masked].astype(int) - data["frames_reset"][masked].astype(int)).max() <= 1
    for s in range(4):
        r.step(_dev(data[f"lanes_{s}"]), _dev(pad_things(data[f"things_{s}"], 64)), stack)
        assert np.abs(stack.cpu().numpy().astype(int) - data[f"frames_{s}"].astype(int)).max() <= 1


def test_fallback_fixture_is_mostly_unclaimed_pixels(pkg, oracle, scenes):
    """Players on portal lines and vertices (engine.py:10956-11171): the frames of the
    upstream renderer, most of whose pixels come from the per-pixel flat fallback."""

    data = load_golden("fallback")
    _sc, blob = scenes("c2", (data["ray_offsets"], data["ray_coscorr"]))
    unowned = oracle.render(blob, data["lanes_0"], data["things_0"])["unowned"]
    assert int(unowned.max()) > 50000 and int(unowned.sum()) > 200000
    r = _renderer(blob, 64)
    _, indexed, _ = r.frames(_dev(data["lanes_0"]), _dev(pad_things(data["things_0"], 64)), indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), data["indexed_0"])


def test_cuda_replays_the_thousand_step_stack(pkg, scenes):
    """c1, 4 lanes, after 1000 agent steps of the upstream engine: the last four
    renders rebuild the upstream four-frame stack (engine.py:9545-9548, 2443-2450)
    within the 1 LSB of its float resize."""

    data = load_golden("c1k")
    _sc, blob = scenes("c1", (data["ray_offsets"], data["ray_coscorr"]))
    r = _renderer(blob, 64)
    n = data["frames"].shape[0]
    stack = torch.zeros((n, 4, 84, 84), dtype=torch.uint8, device=DEV)
    for s in range(4):
        lanes, things = _dev(data[f"stack_lanes_{s}"]), _dev(pad_things(data[f"stack_things_{s}"], 64))
        r.step(lanes, things, stack)
        done = data[f"stack_done_{s}"].astype(bool)
        if done.any():
            r.reset(lanes, things, _dev(done), stack)
    r.check_status()
    assert np.abs(stack.cpu().numpy().astype(int) - data["frames"].astype(int)).max() <= 1


def test_two_renderers_of_different_scenes_side_by_side(pkg, oracle, scenes):
    """A large and a small scene alive on one device, stepped in turns: each keeps
    its own shared-memory size and scratch."""

    from gradoom_b200 import stepper

    sc4, blob4 = scenes("c4")
    sc1, blob1 = scenes("c1")
    big = _renderer(blob4, 8)
    small = _renderer(blob1, 4)
    assert big.shared_bytes != small.shared_bytes
    l4, t4 = stepper.random_lanes(sc4, 6, 8, seed=31)
    l1, t1 = stepper.random_lanes(sc1, 6, 4, seed=32)
    e4, e1 = oracle.render(blob4, l4, t4)["obs"], oracle.render(blob1, l1, t1)["obs"]
    s4 = torch.zeros((6, 4, 84, 84), dtype=torch.uint8, device=DEV)
    s1 = torch.zeros((6, 4, 84, 84), dtype=torch.uint8, device=DEV)
    for _ in range(2):
        big.step(_dev(l4), _dev(t4), s4)
        small.step(_dev(l1), _dev(t1), s1)
    third = _renderer(blob1, 4)          # created after the large one was used
    big.step(_dev(l4), _dev(t4), s4)
    third.step(_dev(l1), _dev(t1), s1)
    torch.cuda.synchronize()
    for r in (big, small, third):
        r.check_status()
    assert np.array_equal(s4[:, 3].cpu().numpy(), e4) and np.array_equal(s4[:, 1].cpu().numpy(), e4)
    assert np.array_equal(s1[:, 3].cpu().numpy(), e1) and np.array_equal(s1[:, 1].cpu().numpy(), e1)


def test_state_packer_kernel_matches_the_fixture_and_the_upstream_frame(pkg, oracle, scenes):
    """gd_pack_state on the engine tensors recorded from the upstream engine (every actor
    class in use, map items included): records equal the fixture's bit for bit, and the
    frame drawn from them is the upstream renderer's (engine.py:14328-14682)."""

    from gradoom_b200 import state as gdstate

    data = load_golden("state")
    _sc, blob = scenes("c1i", (data["ray_offsets"], data["ray_coscorr"]))
    r = _renderer(blob, 64)
    src = engine_from_fixture(data, DEV)
    n = data["lanes_0"].shape[0]
    lanes = torch.zeros((n, 32), dtype=torch.int32, device=DEV)
    things = torch.zeros((n, 64, 4), dtype=torch.int32, device=DEV)
    r.pack_state(gdstate.EngineState(src), lanes, things)
    k = data["things_0"].shape[1]
    assert np.array_equal(lanes.cpu().numpy(), data["lanes_0"])
    assert np.array_equal(things[:, :k].cpu().numpy(), data["things_0"])
    _, indexed, _ = r.frames(lanes, things, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), data["indexed_0"])


@pytest.mark.parametrize("n,seed,items", [(1, 1, 0), (257, 2, 12), (1024, 3, 12)])
def test_state_packer_kernel_matches_the_oracle_packer(n, seed, items, pkg, oracle, scenes):
    """Random engine-shaped states, all classes active: lane and thing records of the
    kernel equal the CPU packer's, twice in a row (the slot-use flags are cleared per call)."""

    from gradoom_b200 import state as gdstate

    _sc, blob = scenes("c1i" if items else "c1")
    r = _renderer(blob, 64)
    lanes = torch.zeros((n, 32), dtype=torch.int32, device=DEV)
    things = torch.zeros((n, 64, 4), dtype=torch.int32, device=DEV)
    for round_ in range(2):
        src = fake_engine(n, seed=seed + 10 * round_, items=items)
        want_lanes, want_things, k = oracle.pack_state(blob, src, 64)
        assert 0 < k <= 64
        dev = fake_engine(n, seed=seed + 10 * round_, items=items, device=DEV)
        things.zero_()
        r.pack_state(gdstate.EngineState(dev), lanes, things)
        r.check_status()
        assert np.array_equal(lanes.cpu().numpy(), want_lanes)
        assert np.array_equal(things.cpu().numpy(), want_things)


def test_state_packer_reports_more_records_than_the_stride(pkg, scenes):
    from gradoom_b200 import native, state as gdstate

    _sc, blob = scenes("c1")
    r = _renderer(blob, 8)
    dev = fake_engine(4, seed=3, device=DEV)
    lanes = torch.zeros((4, 32), dtype=torch.int32, device=DEV)
    things = torch.zeros((4, 8, 4), dtype=torch.int32, device=DEV)
    r.pack_state(gdstate.EngineState(dev), lanes, things)
    assert int(lanes[0, gdstate.L_THINGS]) > 8
    with pytest.raises(native.NativeError):
        r.check_status()


@pytest.mark.parametrize("config", ["c1", "c2"])
def test_kinematics_kernel_follows_the_upstream_trajectories(config, pkg, scenes):
    """gd_player_tics against the per-step player records of the upstream engine (300 steps x
    4 lanes, frame skip 2): bit-equal after every step, and the lane records carry the pose."""

    from gradoom_b200 import state as gdstate

    data = load_golden(f"move_{config}")
    _sc, blob = scenes(config)
    r = _renderer(blob, 4)
    players = _dev(data["players_reset"])
    lanes = torch.zeros((players.shape[0], 32), dtype=torch.int32, device=DEV)
    tics, timeout = int(data["frame_skip"]), int(data["episode_timeout"])
    buttons = _dev(data["buttons"].astype(np.int64)).to(torch.int32)
    for step in range(data["players"].shape[0]):
        r.player_tics(players, buttons[step].contiguous(), tics, timeout, lanes=lanes)
        if step % 25 == 24 or step < 8:
            assert np.array_equal(players.cpu().numpy(), data["players"][step]), f"step {step}"
    final = data["players"][-1]
    assert np.array_equal(players.cpu().numpy(), final)
    got = lanes.cpu().numpy()
    assert np.array_equal(got[:, gdstate.L_X_FIXED], final[:, gdstate.P_X_FIXED])
    assert np.array_equal(got[:, gdstate.L_ANGLE_BAM], final[:, gdstate.P_ANGLE_BAM])
    assert np.array_equal(got[:, gdstate.L_VIEW_Z], final[:, gdstate.P_VIEW_Z])
    assert np.array_equal(got[:, gdstate.L_X].view(np.float32), (final[:, gdstate.P_X_FIXED] / 65536.0).astype(np.float32))


@pytest.mark.parametrize("trial", range(6))
def test_kinematics_kernel_matches_the_oracle_on_random_maps(trial, pkg, oracle):
    """Maps of 2x2 to 16x16 rooms with diagonal lines and floor steps of up to 128 units, 1024 lanes,
    40 steps of 4 tics under random masks over all twenty buttons: the warp-per-lane kernel's player
    records equal the serial CPU restatement's, word for word."""

    from gradoom_b200 import native, scene as gdscene, state as gdstate, stepper

    rng = np.random.default_rng(4400 + trial)
    spec = gdscene.GridSpec(rows=int(rng.integers(2, 17)), cols=int(rng.integers(2, 17)),
                            room=float(rng.choice([96.0, 128.0, 256.0])), seed=700 + trial, wall_textures=4, tex_w=64,
                            tex_h=128, flats=2, floor_max=int(rng.choice([0, 24, 64, 128])), diagonals=bool(trial % 2))
    sc = gdscene.make_grid_scene(spec)
    blob = gdscene.pack_scene(sc)
    n = 1024
    r = native.Renderer(blob, DEV, 1)
    producer = stepper.LaneStepper(sc, n, device=DEV, k_things=0, max_things=1, seed=trial)
    producer.bind_renderer(r)
    producer.reset(torch.ones(n, dtype=torch.bool, device=DEV), torch.arange(n, device=DEV) + 1)
    players = producer.players.clone()
    start = players.cpu().numpy().copy()
    want = start.copy()
    for step in range(40):
        masks = rng.integers(0, 1 << 20, size=n).astype(np.uint32)
        if step % 3:
            masks &= np.uint32(0b111111110)          # mostly the movement buttons, so that the players get somewhere
        r.player_tics(players, _dev(masks.astype(np.int64)).to(torch.int32), 4, 4200)
        oracle.player_tics(blob, want, masks, 4, 4200)
    r.close()
    assert np.array_equal(players.cpu().numpy(), want)
    assert (want[:, gdstate.P_X_FIXED] != start[:, gdstate.P_X_FIXED]).mean() > 0.9


def test_kinematics_kernel_matches_the_oracle_on_a_seeded_batch(pkg, oracle, scenes):
    """2048 lanes of c2 walking for 30 steps under random buttons with solid monsters
    around: the kernel's player records equal the CPU restatement's."""

    from conftest import fake_engine
    from gradoom_b200 import state as gdstate, stepper

    sc, blob = scenes("c2")
    n = 2048
    r = _renderer(blob, 12)
    producer = stepper.LaneStepper(sc, n, device=DEV, k_things=12, max_things=12, seed=3)
    producer.bind_renderer(r)
    producer.reset(torch.ones(n, dtype=torch.bool, device=DEV), torch.arange(n, device=DEV) + 1)
    players = producer.players.clone()
    want = players.cpu().numpy().copy()
    monsters = fake_engine(n, seed=77, span=1900.0)
    monsters.enemy_z = torch.zeros_like(monsters.enemy_z) + 8.0
    dev_monsters = fake_engine(n, seed=77, span=1900.0, device=DEV)
    dev_monsters.enemy_z = torch.zeros_like(dev_monsters.enemy_z) + 8.0
    solid_dev = gdstate.SolidActors(dev_monsters)
    rng = np.random.default_rng(5)
    for step in range(30):
        masks = rng.integers(0, 1 << 9, size=n).astype(np.uint32) & np.uint32(0b111111110)
        r.player_tics(players, _dev(masks.astype(np.int64)).to(torch.int32), 2, 4200, actors=solid_dev)
        oracle.player_tics(blob, want, masks, 2, 4200, actors=monsters)
    assert np.array_equal(players.cpu().numpy(), want)
    moved = (want[:, gdstate.P_X_FIXED] != producer.players.cpu().numpy()[:, gdstate.P_X_FIXED]).mean()
    assert moved > 0.9


def test_full_size_batch_properties(pkg, oracle, scenes):
    """4096 lanes on the 64-sector map: size-independent properties plus an
    oracle check of a lane sample."""

    from gradoom_b200 import stepper

    sc, blob = scenes("c2")
    n, k = 4096, 12
    lanes, things = stepper.random_lanes(sc, n, k, seed=11)
    r = _renderer(blob, k)
    dl, dt = _dev(lanes), _dev(things)
    stack = torch.zeros((n, 4, 84, 84), dtype=torch.uint8, device=DEV)
    r.reset(dl, dt, torch.ones(n, dtype=torch.bool, device=DEV), stack)
    first = stack.clone()
    assert torch.equal(first[:, 0], first[:, 3])           # fill: all slots equal
    r.step(dl, dt, stack)
    assert torch.equal(stack[:, :3], first[:, 1:])          # roll moved the old slots down
    assert torch.equal(stack[:, 3], first[:, 3])            # same state, same frame: deterministic
    obs, _, _ = r.frames(dl, dt, obs=True)
    assert torch.equal(obs, stack[:, 3])                    # stateless call agrees with the stack path
    r.check_status()
    sample = np.arange(0, n, 97)
    expected = oracle.render(blob, lanes[sample], things[sample])["obs"]
    assert np.array_equal(obs.cpu().numpy()[sample], expected)
    # idempotence of a fill with an all-false mask
    before = stack.clone()
    r.reset(dl, dt, torch.zeros(n, dtype=torch.bool, device=DEV), stack)
    assert torch.equal(stack, before)


def test_known_answer_sprite_scenes(pkg):
    import kat
    from gradoom_b200 import scene as gdscene

    sc, (lanes, things), expected = kat.transparent_case()
    r = _renderer(gdscene.pack_scene(sc), things.shape[1])
    _, indexed, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
    assert indexed[0, 103, 160].item() == expected


def test_abi_argument_validation(pkg, scenes):
    from gradoom_b200 import native, stepper

    sc, blob = scenes("c1")
    r = _renderer(blob, 4)
    lanes, things = stepper.random_lanes(sc, 4, 4, seed=1)
    dl, dt = _dev(lanes), _dev(things)
    stack = torch.zeros((4, 4, 84, 84), dtype=torch.uint8, device=DEV)
    lib = native.load()
    stream = torch.cuda.current_stream().cuda_stream
    # too little scratch
    rc = lib.gd_render_step(r.handle, dl.data_ptr(), dt.data_ptr(), 4, 1, stack.data_ptr(), r.scratch.data_ptr(),
                            16, r.status.data_ptr(), stream)
    assert rc == -7
    # misaligned pointer
    rc = lib.gd_render_step(r.handle, dl.data_ptr() + 4, dt.data_ptr(), 4, 1, stack.data_ptr(),
                            r.scratch.data_ptr(), r.scratch_bytes, r.status.data_ptr(), stream)
    assert rc == -5
    # null stack, negative n, empty batch
    assert lib.gd_render_step(r.handle, dl.data_ptr(), dt.data_ptr(), 4, 1, None, r.scratch.data_ptr(),
                              r.scratch_bytes, r.status.data_ptr(), stream) == -1
    assert lib.gd_render_step(r.handle, dl.data_ptr(), dt.data_ptr(), -1, 1, stack.data_ptr(),
                              r.scratch.data_ptr(), r.scratch_bytes, r.status.data_ptr(), stream) == -4
    assert lib.gd_render_step(r.handle, dl.data_ptr(), dt.data_ptr(), 0, 1, stack.data_ptr(),
                              r.scratch.data_ptr(), r.scratch_bytes, r.status.data_ptr(), stream) == 0
    # a renderer bound to another device than the current one
    if torch.cuda.device_count() > 1:
        with torch.cuda.device(1):
            assert lib.gd_render_step(r.handle, dl.data_ptr(), dt.data_ptr(), 4, 1, stack.data_ptr(),
                                      r.scratch.data_ptr(), r.scratch_bytes, r.status.data_ptr(), stream) == -10
    # a corrupted blob header is refused
    bad = blob.copy()
    bad[:4] = 0
    handle = ctypes.c_void_p()
    assert lib.gd_renderer_create(bad.ctypes.data, r.blob.data_ptr(), bad.size, 0, 4, ctypes.byref(handle)) == -2
    with pytest.raises(ValueError):
        r.step(dl.to(torch.int64), dt, stack)
    with pytest.raises(TypeError):
        r.step(dl.cpu(), dt, stack)
    torch.cuda.synchronize()


def test_thing_overflow_sets_the_status_word(pkg, scenes):
    from gradoom_b200 import native, stepper, state as gdstate

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 2, 4, seed=1)
    lanes[:, gdstate.L_THINGS] = 9          # claims more records than the stride holds
    r = _renderer(blob, 4)
    r.frames(_dev(lanes), _dev(things), obs=True)
    with pytest.raises(native.NativeError):
        r.check_status()
    r.frames(_dev(stepper.random_lanes(sc, 2, 4, seed=1)[0]), _dev(things), obs=True)
    r.check_status()                        # cleared after being reported


def test_unclaimed_pixels_show_the_flat_fallback(pkg, oracle, scenes):
    """Lanes in which some pixels are claimed by no seg and no visplane: those
    pixels come from the per-pixel flat fallback (engine.py:10956-11171)."""

    from gradoom_b200 import stepper

    sc, blob = scenes("c2")
    lanes, things = stepper.random_lanes(sc, 512, 12, seed=11)
    expected = oracle.render(blob, lanes, things)
    chosen = np.flatnonzero(expected["unowned"] > 0)
    assert len(chosen) >= 4, "the seeded batch is expected to contain such lanes"
    r = _renderer(blob, 12)
    _, indexed, _ = r.frames(_dev(lanes[chosen]), _dev(things[chosen]), indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"][chosen])


@pytest.mark.gpu
def test_flat_fallback_after_free_movement(pkg, oracle, scenes):
    """Players that have walked freely stand on or next to portal lines now and
    then; their frames need the fallback's vertical and horizontal repairs."""

    from gradoom_b200 import state as gdstate, stepper

    sc, blob = scenes("c2")
    n = 512
    lanes, things = stepper.random_lanes(sc, n, 12, seed=1000)
    # every eighth player is moved onto a portal line of the grid or a hair beside it
    rng = np.random.default_rng(7)
    moved = np.arange(0, n, 8)
    offsets = rng.choice(np.asarray([0.0, 1.0 / 65536, -1.0 / 65536, 0.25, -0.25, 1.0]), size=len(moved))
    x = (rng.integers(1, 8, size=len(moved)) * 256 + offsets).astype(np.float32)
    lanes[moved, gdstate.L_X] = x.view(np.int32)
    lanes[moved, gdstate.L_X_FIXED] = np.round(x.astype(np.float64) * 65536).astype(np.int32)
    expected = oracle.render(blob, lanes, things)
    chosen = np.flatnonzero(expected["unowned"] > 0)
    assert len(chosen) >= 4, "the seeded batch is expected to contain such lanes"
    r = _renderer(blob, 12)
    _, indexed, _ = r.frames(_dev(lanes[chosen]), _dev(things[chosen]), indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"][chosen])


@pytest.mark.gpu
def test_step_with_frames_equals_step_plus_frames(pkg, scenes):
    """The fused entry point pushes the same stack as gd_render_step and writes
    the same frames as gd_render_frames."""

    import torch

    from gradoom_b200 import stepper

    sc, blob = scenes("c3")
    lanes, things = stepper.random_lanes(sc, 96, 12, seed=5)
    r = _renderer(blob, 12)
    dl, dt = _dev(lanes), _dev(things)
    base = torch.randint(0, 256, (96, 4, 84, 84), dtype=torch.uint8, device="cuda")
    a, b = base.clone(), base.clone()
    r.step(dl, dt, a)
    _, indexed, rgb = r.frames(dl, dt, indexed=True, rgb=True)
    indexed2, rgb2 = torch.empty_like(indexed), torch.empty_like(rgb)
    r.step_frames(dl, dt, b, indexed=indexed2, rgb=rgb2)
    r.check_status()
    assert torch.equal(a, b)
    assert torch.equal(indexed, indexed2)
    assert torch.equal(rgb, rgb2)


@pytest.mark.gpu
@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_step_matches_device_step(pkg, scenes, pinned):
    """gd_render_step_host, with a pinned result buffer (written by the kernel
    itself) and with a pageable one (chunked copies), against gd_render_step."""

    import torch

    from gradoom_b200 import stepper

    sc, blob = scenes("c1")
    n = 2304                                   # enough lanes for the chunked path, not a multiple of the chunk size
    lanes, things = stepper.random_lanes(sc, n, 4, seed=21)
    r = _renderer(blob, 4)
    dl, dt = _dev(lanes), _dev(things)
    base = torch.randint(0, 256, (n, 4, 84, 84), dtype=torch.uint8, device="cuda")
    expect, got = base.clone(), base.clone()
    r.step(dl, dt, expect)
    host_lanes, host_things = torch.from_numpy(lanes), torch.from_numpy(things)
    host_obs = torch.zeros((n, 84, 84), dtype=torch.uint8)
    if pinned:
        host_lanes, host_things, host_obs = host_lanes.pin_memory(), host_things.pin_memory(), host_obs.pin_memory()
    r.step_host(host_lanes, host_things, torch.empty_like(dl), torch.empty_like(dt), got, host_obs)
    torch.cuda.synchronize()
    r.check_status()
    assert torch.equal(expect, got)
    assert torch.equal(host_obs, expect[:, 3].cpu())


@pytest.mark.gpu
def test_screen_flashes_blend_rgb_and_observation(pkg, oracle):
    """Lanes that ask for the damage / bonus screen blends (engine.py:15385-15397):
    RGB24 bit-exact against the upstream fixture, observation equal to the oracle's
    and within 1 LSB of the upstream float path; plain lanes drawn afterwards by
    the same CTAs get the plain palette back."""

    import torch

    from gradoom_b200 import scene as gdscene

    data = load_golden("flashes")
    sc = gdscene.make_grid_scene(gdscene.GRID_CONFIGS["c1"])
    sc.meta["damage_alpha"] = data["damage_alpha"]
    blob = gdscene.pack_scene(sc, ray_table_override=(data["ray_offsets"], data["ray_coscorr"]))
    k = max(data[f"things_{ci}"].shape[1] for ci in range(3))
    r = _renderer(blob, k)
    for ci in range(3):
        lanes, things = data[f"lanes_{ci}"], pad_things(data[f"things_{ci}"], k)
        expected = oracle.render(blob, lanes, things, mask_hud=True)
        obs, _, rgb = r.frames(_dev(lanes), _dev(things), obs=True, rgb=True)
        r.check_status()
        assert np.array_equal(rgb.cpu().numpy(), data[f"rgb_{ci}"])
        assert np.array_equal(obs.cpu().numpy(), expected["obs"])
        assert np.abs(obs.cpu().numpy().astype(int) - data[f"obs_float_{ci}"].astype(int)).max() <= 1
    # blended and plain lanes interleaved in one launch
    lanes = np.concatenate([data["lanes_2"], data["lanes_2"]])
    lanes[4:, 8] &= 3
    things = np.concatenate([pad_things(data["things_2"], k)] * 2)
    order = np.array([0, 4, 1, 5, 2, 6, 3, 7] * 40)
    _, _, rgb = r.frames(_dev(lanes[order]), _dev(things[order]), rgb=True)
    want = oracle.rgb(blob, oracle.render(blob, lanes, things)["indexed"], lanes)[order]
    assert np.array_equal(rgb.cpu().numpy(), want)


@pytest.mark.gpu
def test_player_exactly_on_a_portal_line(pkg, oracle, scenes):
    """A recorded c2 lane whose player stands on a room boundary (x = 1792 - 2^-15):
    no seg claims 84 % of the view, so the frame is mostly flat fallback and the
    pixel queue is refilled many times."""

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "lane_on_portal_line.npz"))
    sc, blob = scenes("c2")
    lanes, things = data["lanes"], data["things"]
    expected = oracle.render(blob, lanes, things)
    assert expected["unowned"][0] > 50000
    r = _renderer(blob, things.shape[1])
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])


@pytest.mark.gpu
def test_sixty_four_things_per_lane_and_empty_batches(pkg, oracle, scenes):
    """The per-column candidate mask is 64 bits wide: lanes with exactly 64 things,
    most of them crowded into one room so that many overlap in a column; and a
    launch over zero lanes touches nothing."""

    import torch

    from gradoom_b200 import stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 24, 64, seed=31)
    tf = things.view(np.float32)
    room = float(sc.meta["spec"].room)
    tf[:, 8:, 0] = tf[:, 8:, 0] % room + room       # things 8..63 share the second room of the first row
    tf[:, 8:, 1] = tf[:, 8:, 1] % room
    floor = sc.sector_heights[1, 0]
    tf[:, 8:, 2] = floor
    expected = oracle.render(blob, lanes, things)
    r = _renderer(blob, 64)
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])
    stack = torch.full((0, 4, 84, 84), 7, dtype=torch.uint8, device="cuda")
    r.step(_dev(lanes[:0]), _dev(things[:0]), stack)
    r.check_status()


@pytest.mark.gpu
def test_render_step_captures_into_a_cuda_graph(pkg, scenes):
    """The entry points allocate nothing and never synchronise, so a step can be
    captured once and replayed on new records written into the same buffers."""

    import torch

    from gradoom_b200 import stepper

    sc, blob = scenes("c1")
    la, ta = stepper.random_lanes(sc, 300, 4, seed=41)
    lb, tb = stepper.random_lanes(sc, 300, 4, seed=42)
    r = _renderer(blob, 4)
    lanes, things = _dev(la), _dev(ta)
    stack = torch.zeros((300, 4, 84, 84), dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        r.step(lanes, things, stack)                 # warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        r.step(lanes, things, stack)
    stack.zero_()
    expect = torch.zeros_like(stack)
    for records in ((la, ta), (lb, tb), (la, ta)):
        lanes.copy_(_dev(records[0])); things.copy_(_dev(records[1]))
        graph.replay()
        r.step(_dev(records[0]), _dev(records[1]), expect)
    torch.cuda.synchronize()
    r.check_status()
    assert torch.equal(stack, expect)
    assert not torch.equal(stack[:, 3], stack[:, 2])


@pytest.mark.parametrize("name", ["decals_c1d", "decals_c4d", "decals_c1md", "decals_fallback"])
def test_cuda_draws_the_upstream_bullet_chips(name, pkg, oracle, scenes):
    """The decal layer (engine.py:13747-13991) against the frames recorded from the upstream engine."""

    from conftest import decal_rings

    data = load_golden(name)
    _sc, blob = scenes(str(data["config"]), (data["ray_offsets"], data["ray_coscorr"]))
    r = _renderer(blob, 64)
    lanes, things = _dev(data["lanes_0"]), _dev(pad_things(data["things_0"], 64))
    r.bind_decals(_dev(decal_rings(data)))
    _, indexed, _ = r.frames(lanes, things, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), data["indexed_0"])
    r.bind_decals(None)
    _, bare, _ = r.frames(lanes, things, indexed=True)
    assert int((bare.cpu().numpy() != data["indexed_0"]).sum()) == int(data["changed_pixels"])


@pytest.mark.parametrize("name,n,k,per_lane,slots,seed", [("c4d", 96, 8, 60, 1024, 1), ("c1d", 64, 4, 200, 256, 2),
                                                          ("c1d", 5, 0, 1, 1, 3)])
def test_cuda_decals_match_the_oracle_on_seeded_lanes(name, n, k, per_lane, slots, seed, pkg, oracle, scenes):
    from gradoom_b200 import stepper

    sc, blob = scenes(name)
    lanes, things = stepper.random_lanes(sc, n, k, seed=seed)
    rings = stepper.random_decals(sc, lanes, per_lane, slots, seed=seed + 100)
    expected = oracle.render(blob, lanes, things, decals=rings.view(oracle.DECAL_DTYPE)[..., 0])
    bare = oracle.render(blob, lanes, things)
    if per_lane > 1:
        assert int((expected["indexed"] != bare["indexed"]).sum()) > 1000
    r = _renderer(blob, k)
    r.bind_decals(_dev(rings))
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])


def test_decal_rings_are_ignored_by_a_scene_without_chip_bitmaps(pkg, oracle, scenes):
    from gradoom_b200 import native, stepper

    sc, blob = scenes("c1")
    lanes, things = stepper.random_lanes(sc, 8, 4, seed=5)
    rings = stepper.random_decals(sc, lanes, 30, 64, seed=6)
    r = _renderer(blob, 4)
    _, bare, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
    r.bind_decals(_dev(rings))
    _, bound, _ = r.frames(_dev(lanes), _dev(things), indexed=True)
    assert torch.equal(bare, bound)
    with pytest.raises(native.NativeError):
        r.bind_decals(torch.zeros((8, 2048, 4), dtype=torch.int32, device=DEV))     # more slots than the renderer accepts
    with pytest.raises(ValueError):
        r.bind_decals(torch.zeros((8, 64, 3), dtype=torch.int32, device=DEV))
    r.bind_decals(_dev(rings[:4]))                     # rings for four lanes, a call that draws eight
    with pytest.raises(ValueError):
        r.frames(_dev(lanes), _dev(things), indexed=True)


def test_cuda_draws_a_scene_compiled_from_wad_files(pkg, oracle):
    """WAD + UDMF in (src/gradoom/scenario.py:457-1064), frames out: textures composed from patches,
    sprites with mirrored rotations, weapon and status-bar pictures, all through the blob."""

    import wadgen
    from gradoom_b200 import scene as gdscene, state as gdstate, wad as gdwad

    sc = gdscene.from_compiled_scenario(gdwad.compile_scenario(*wadgen.synthetic_pair(gdscene, gdwad)))
    blob = gdscene.pack_scene(sc)
    rng = np.random.default_rng(8)
    poses = [(float(rng.uniform(40, 980)), float(rng.uniform(40, 980)), float(rng.uniform(0, 6.28))) for _ in range(24)]
    poses = [(x + (20 if x % 256 < 20 else 0) - (20 if x % 256 > 236 else 0),
              y + (20 if y % 256 < 20 else 0) - (20 if y % 256 > 236 else 0), a) for x, y, a in poses]
    lanes = wadgen.view_lanes(gdscene, gdstate, sc, poses)
    k = 6
    things = np.zeros((len(poses), k, 4), dtype=np.int32)
    tf = things.view(np.float32)
    for i in range(len(poses)):
        for j in range(k):
            x, y = float(rng.uniform(40, 980)), float(rng.uniform(40, 980))
            sector = gdscene.sector_at(sc, np.float32([x]), np.float32([y]))[0]
            tf[i, j, 0], tf[i, j, 1], tf[i, j, 2] = x, y, sc.sector_heights[sector, 0]
            word = int(rng.integers(0, len(sc.spr_atlas))) | (gdstate.THING_ALIVE << 16) | (0xFF << 24)   # style -1
            things[i, j, 3] = np.uint32(word).view(np.int32)
    lanes[:, gdstate.L_THINGS] = k
    expected = oracle.render(blob, lanes, things, mask_hud=False)
    r = _renderer(blob, k)
    obs, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True, mask_hud=False)
    r.check_status()
    assert np.array_equal(indexed.cpu().numpy(), expected["indexed"])
    assert np.array_equal(obs.cpu().numpy(), expected["obs"])


def test_device_libm_against_the_hosts_on_the_renderers_arguments(pkg):
    """The float32 transcendentals of the path (engine.py:14684-14688, 13994-14009, 10966-10974) run in
    the device's libm here; the reference runs them in ATen: its CUDA kernels on a GPU, its CPU kernels
    (which recorded the fixtures) on the host.  On arguments formed the way the renderer forms them
    this counts how often the library's calls differ from either, bounds the distance, and checks that
    the quantities derived from them (sprite depth, rotation step) agree.  With GD_LIBM_LOG set the
    counts are appended to that file."""

    import json
    import math

    from gradoom_b200 import native

    g = torch.Generator().manual_seed(77)
    n = 1 << 20
    # positions on the 16.16 grid of a 2048-unit map: thing minus player
    px = torch.randint(0, 2048 << 16, (n,), generator=g).to(torch.float32) / 65536.0
    py = torch.randint(0, 2048 << 16, (n,), generator=g).to(torch.float32) / 65536.0
    tx = torch.randint(0, 2048 << 16, (n,), generator=g).to(torch.float32) / 65536.0
    ty = torch.randint(0, 2048 << 16, (n,), generator=g).to(torch.float32) / 65536.0
    dx, dy = tx - px, ty - py
    view = torch.randint(0, 1 << 32, (n,), generator=g).to(torch.float32) * (2.0 * math.pi / float(1 << 32))

    def ulps(a, b):
        ia, ib = a.view(torch.int32).to(torch.int64), b.view(torch.int32).to(torch.int64)
        ia = torch.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
        ib = torch.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
        return (ia - ib).abs()

    def compare(ours, aten_cpu, aten_cuda):
        d = ulps(aten_cpu, ours)
        return {"n": n, "differ_from_aten_cpu": int((d > 0).sum()), "max_ulp_from_aten_cpu": int(d.max()),
                "differ_from_aten_cuda": int((ulps(aten_cuda.cpu(), ours) > 0).sum())}

    report = {}
    host_bearing = torch.atan2(dy, dx)
    dev_bearing = native.probe_libm(native.PROBE_ATAN2F, dy.to(DEV), dx.to(DEV)).cpu()
    report["atan2f"] = compare(dev_bearing, host_bearing, torch.atan2(dy.to(DEV), dx.to(DEV)))
    rel = torch.remainder(host_bearing - view + math.pi, 2 * math.pi) - math.pi
    for name, fn, op in (("cosf", native.PROBE_COSF, torch.cos), ("sinf", native.PROBE_SINF, torch.sin)):
        report[name] = compare(native.probe_libm(fn, rel.to(DEV)).cpu(), op(rel), op(rel.to(DEV)))
    squares = dx * dx + dy * dy
    dev_dist = native.probe_libm(native.PROBE_HYPOT, dx.to(DEV), dy.to(DEV)).cpu()
    report["sqrtf"] = compare(dev_dist, torch.sqrt(squares), torch.sqrt(squares.to(DEV)))
    exact = torch.sqrt(squares.to(torch.float64)).to(torch.float32)       # the correctly rounded root
    report["sqrtf"]["differ_from_correctly_rounded"] = int((dev_dist != exact).sum())
    report["sqrtf"]["aten_cpu_differs_from_correctly_rounded"] = int((torch.sqrt(squares) != exact).sum())
    # derived quantities: sprite depth (dist * cos(rel)) and the sprite rotation step of eight
    dev_rel = torch.remainder(dev_bearing - view + math.pi, 2 * math.pi) - math.pi
    host_depth = torch.sqrt(squares) * torch.cos(rel)
    dev_depth = dev_dist * native.probe_libm(native.PROBE_COSF, dev_rel.to(DEV)).cpu()
    close = (host_depth - dev_depth).abs() <= 1e-4 * dev_dist.clamp_min(1.0)
    report["sprite_depth"] = {"n": n, "differ_from_aten_cpu": int((host_depth != dev_depth).sum()),
                              "beyond_1e-4_relative": int((~close).sum())}
    facing = torch.rand(n, generator=g) * 2 * math.pi

    def rotation(bearing):
        relative = torch.remainder(bearing + math.pi - facing + math.pi / 8, 2 * math.pi)
        return torch.remainder(torch.floor(relative / (math.pi / 4)), 8)

    report["sprite_rotation_step"] = {"n": n, "differ_from_aten_cpu": int((rotation(host_bearing) != rotation(dev_bearing)).sum())}
    log = os.environ.get("GD_LIBM_LOG")
    if log:
        with open(log, "a") as f:
            f.write(json.dumps(report) + "\n")
    for name in ("atan2f", "cosf", "sinf", "sqrtf"):
        assert report[name]["max_ulp_from_aten_cpu"] <= 4
    assert report["sqrtf"]["differ_from_correctly_rounded"] == 0     # IEEE square root, products and sum rounded separately
    assert report["sprite_depth"]["beyond_1e-4_relative"] == 0
    assert report["sprite_rotation_step"]["differ_from_aten_cpu"] <= n // 10000


@pytest.mark.parametrize("name,n,k", [("c2", 300, 12), ("c4", 160, 32), ("c1m", 64, 4)])
def test_observation_only_calls_equal_full_frame_calls(name, n, k, pkg, oracle, scenes):
    """A call that draws no status bar and returns no full frame keeps only the view rows of the frame
    on chip and stages other tables than a full-frame call does; the observations must not differ."""

    from gradoom_b200 import stepper

    sc, blob = scenes(name)
    lanes, things = stepper.random_lanes(sc, n, k, seed=31)
    r = _renderer(blob, k)
    assert r.shared_bytes - 32 * 320 <= r.shared_bytes_view <= r.shared_bytes + 16384   # 10 KB of frame out, tables in
    view_only, _, _ = r.frames(_dev(lanes), _dev(things), obs=True, mask_hud=True)
    full, indexed, _ = r.frames(_dev(lanes), _dev(things), obs=True, indexed=True, mask_hud=True)
    r.check_status()
    assert torch.equal(view_only, full)
    expected = oracle.render(blob, lanes[:32], things[:32], mask_hud=True)
    assert np.array_equal(view_only[:32].cpu().numpy(), expected["obs"])
    assert np.array_equal(indexed[:32, :208].cpu().numpy(), expected["indexed"][:, :208])
    stack = torch.zeros((n, 4, 84, 84), dtype=torch.uint8, device=DEV)
    r.step(_dev(lanes), _dev(things), stack)
    assert torch.equal(stack[:, 3], full)
