"""The GraDoomVecEnv mirror: tensor contracts and error behaviour of the
reference's device API (src/gradoom/env.py:851-942, 1037-1066; upstream
tests/test_env.py:109-242, tests/test_turbo_api_contract.py:326-349, 509-519)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _env(scenes, n=6, **kw):
    from gradoom_b200 import env as gdenv

    sc, _ = scenes("c1")
    timeout = kw.pop("episode_timeout", None)
    if timeout is not None:
        kw["vizdoom_config"] = {"episode_timeout": timeout}
    return gdenv.GraDoomVecEnv(compiled_scenario=sc, num_envs=n, device=DEV, max_things=8, frame_skip=2,
                               obs_crop=(0, 32, 0, 0), obs_crop_mode="mask", **kw)


def test_reset_and_step_contracts(pkg, oracle, scenes):
    e = _env(scenes, render_mode="rgb_array")
    n = e.num_envs
    lane = torch.arange(n, device=DEV)
    obs, signals = e.reset_device(torch.ones(n, dtype=torch.bool, device=DEV), lane + 1)
    assert obs.shape == (n, 4, 84, 84) and obs.dtype == torch.uint8 and obs.device == DEV
    assert signals.shape == (n, 27) and signals.dtype == torch.float32
    assert torch.equal(obs[:, 0], obs[:, 3])
    t = e.step_device(torch.full((n,), 7, device=DEV, dtype=torch.int64))
    assert t.observations.data_ptr() == obs.data_ptr()            # live view of the stack buffer
    assert t.rewards.shape == (n,) and t.terminated.dtype == torch.bool and t.truncated.dtype == torch.bool
    # what the env shows equals the oracle's rendering of the producer's state
    lanes, things = e._producer.render_inputs()
    from gradoom_b200 import scene as gdscene

    expected = oracle.render(gdscene.pack_scene(e.scene), lanes.cpu().numpy(), things.cpu().numpy())["obs"]
    assert np.array_equal(t.observations[:, 3].cpu().numpy(), expected)
    a = e.step_and_reset_device(torch.zeros(n, device=DEV, dtype=torch.int32), lane + 100)
    assert a.final_observations.data_ptr() != a.observations.data_ptr()
    assert torch.equal(a.final_observations, a.observations)      # nobody was done: identical content
    frame = e.render()
    assert isinstance(frame, np.ndarray) and frame.shape == (240, 320, 3) and frame.dtype == np.uint8
    assert len(e.get_images()) == n
    e.check_status()
    e.close()
    e.close()
    with pytest.raises(RuntimeError):
        e.render()
    with pytest.raises(RuntimeError):
        e.step_device(torch.zeros(n, device=DEV, dtype=torch.int64))


def test_masked_reset_preserves_other_lanes(pkg, scenes):
    e = _env(scenes)
    n = e.num_envs
    lane = torch.arange(n, device=DEV)
    e.reset_device(torch.ones(n, dtype=torch.bool, device=DEV), lane + 1)
    for a in (2, 6, 2):
        e.step_device(torch.full((n,), a, device=DEV, dtype=torch.int64))
    before = e.step_device(torch.full((n,), 2, device=DEV, dtype=torch.int64)).observations.clone()
    mask = torch.zeros(n, dtype=torch.bool, device=DEV)
    mask[1] = True
    obs, _ = e.reset_device(mask, lane + 50)
    assert torch.equal(obs[0], before[0]) and torch.equal(obs[2:], before[2:])
    assert torch.equal(obs[1, 0], obs[1, 3]) and not torch.equal(obs[1], before[1])
    e.close()


def test_timeouts_trigger_the_on_device_auto_reset(pkg, scenes):
    e = _env(scenes, n=4, episode_timeout=7)
    n = e.num_envs
    lane = torch.arange(n, device=DEV)
    e.reset_device(torch.ones(n, dtype=torch.bool, device=DEV), lane + 1)
    done_seen = False
    for step in range(5):
        t = e.step_and_reset_device(torch.full((n,), 6, device=DEV, dtype=torch.int64), lane + 10 * (step + 1))
        if bool(t.truncated.any()):
            done_seen = True
            assert torch.equal(t.observations[:, 0], t.observations[:, 3])      # refilled stack
            assert not torch.equal(t.final_observations, t.observations)
            break
    assert done_seen
    e.close()


def test_validation_errors(pkg, scenes):
    e = _env(scenes, n=4)
    n = 4
    good = torch.zeros(n, device=DEV, dtype=torch.int64)
    with pytest.raises(TypeError):
        e.step_device([0, 0, 0, 0])
    with pytest.raises(TypeError):
        e.step_device(good.cpu())
    with pytest.raises(ValueError):
        e.step_device(torch.zeros(n + 1, device=DEV, dtype=torch.int64))
    with pytest.raises(TypeError):
        e.step_device(torch.zeros(n, device=DEV, dtype=torch.float32))
    with pytest.raises(TypeError):
        e.reset_device(torch.ones(n, device=DEV, dtype=torch.uint8), good)
    with pytest.raises(RuntimeError):
        e.step(good)                                   # lanes were never reset
    e.reset_device(torch.ones(n, dtype=torch.bool, device=DEV), good + 1)
    with pytest.raises(ValueError):
        e.step(torch.full((n,), 17, device=DEV, dtype=torch.int64))
    assert e.render() is None                          # render_mode None
    assert e.get_images() == [None] * n
    with pytest.raises(TypeError):
        e.render_lane(True)
    with pytest.raises(IndexError):
        e.render_lane(n)
    hwc = _env(scenes, n=2, obs_layout="hwc")
    obs, _ = hwc.reset_device(torch.ones(2, dtype=torch.bool, device=DEV), torch.ones(2, device=DEV, dtype=torch.int64))
    assert obs.shape == (2, 84, 84, 4)
    e.close()
    hwc.close()


@pytest.mark.gpu
def test_ring_stack_policy_shows_the_same_windows_as_the_rolled_stack(pkg, scenes):
    """Two environments with the same seeds, one keeping the reference's rolled stack and one the
    mirrored ring: observations equal after every reset and step, including masked auto-resets."""

    import torch

    from gradoom_b200.env import GraDoomVecEnv

    sc, _ = scenes("c1")
    n = 96
    envs = [GraDoomVecEnv(compiled_scenario=sc, num_envs=n, device="cuda", max_things=8, frame_skip=2,
                          obs_crop=(0, 32, 0, 0), obs_crop_mode="mask", vizdoom_config={"episode_timeout": 10},
                          producer_seed=3, stack_policy=p)
            for p in ("roll", "ring")]
    everyone = torch.ones(n, dtype=torch.bool, device="cuda")
    seeds = torch.arange(n, device="cuda") + 1
    first = [e.reset_device(everyone, seeds)[0] for e in envs]
    assert torch.equal(first[0], first[1]) and tuple(first[1].shape) == (n, 4, 84, 84)
    g = torch.Generator(device="cuda").manual_seed(4)
    for step in range(11):
        actions = torch.randint(0, 17, (n,), device="cuda", generator=g)
        if step == 5:                        # a masked reset of a third of the lanes between steps
            mask = (torch.arange(n, device="cuda") % 3) == 0
            partial = [e.reset_device(mask, seeds + 100)[0] for e in envs]
            assert torch.equal(partial[0], partial[1])
        out = [e.step_and_reset_device(actions, seeds + 1000 * (step + 1)) for e in envs]
        assert torch.equal(out[0].observations, out[1].observations), step
        assert torch.equal(out[0].final_observations, out[1].final_observations), step
    hwc = GraDoomVecEnv(compiled_scenario=sc, num_envs=4, device="cuda", max_things=8, frame_skip=2,
                        obs_crop=(0, 32, 0, 0), obs_crop_mode="mask", obs_layout="hwc", stack_policy="ring")
    assert tuple(hwc.reset_device(torch.ones(4, dtype=torch.bool, device="cuda"), seeds[:4])[0].shape) == (4, 84, 84, 4)
    for e in envs + [hwc]:
        e.check_status()
        e.close()


@pytest.mark.gpu
def test_engine_state_producer_packs_on_the_device(pkg, oracle, scenes):
    """``EngineStateProducer`` around an object with the reference engine's tensors and
    methods: the environment's observations are the oracle's render of the oracle-packed
    state, after reset and after a step that changes the state."""

    from conftest import fake_engine
    from gradoom_b200 import env as gdenv

    sc, blob = scenes("c1")
    n = 5

    class Engine:
        """The slice of the reference engine's interface the producer drives."""

        def __init__(self):
            self.__dict__.update(vars(fake_engine(n, seed=21, device="cuda:0")))
            self.signal_buffer = torch.zeros((n, 27), device="cuda:0")
            self.pending_reset = torch.zeros(n, dtype=torch.bool, device="cuda:0")
            self.render_frame = None
            self.steps = 0

        def reset(self, mask, seeds):
            self.render_frame(mask)

        def step(self, buttons):
            self.render_frame()
            self.steps += 1
            self.__dict__.update(vars(fake_engine(n, seed=21 + self.steps, device="cuda:0")))
            zeros = torch.zeros(n, device="cuda:0")
            return None, zeros, zeros.bool(), zeros.bool()

    engine = Engine()
    producer = gdenv.EngineStateProducer(engine, sc, 64)
    e = gdenv.GraDoomVecEnv(compiled_scenario=sc, num_envs=n, device="cuda:0", producer=producer, max_things=64,
                            frame_skip=2, obs_crop=(0, 32, 0, 0), obs_crop_mode="mask")
    obs, _signals = e.reset_device(torch.ones(n, dtype=torch.bool, device="cuda:0"),
                                   torch.arange(n, device="cuda:0"))
    lanes, things, _k = oracle.pack_state(blob, fake_engine(n, seed=21), 64)
    want = oracle.render(blob, lanes, things)["obs"]
    assert np.array_equal(obs[:, 3].cpu().numpy(), want) and np.array_equal(obs[:, 0].cpu().numpy(), want)
    t = e.step_device(torch.zeros(n, dtype=torch.int64, device="cuda:0"))
    lanes, things, _k = oracle.pack_state(blob, fake_engine(n, seed=22), 64)
    assert np.array_equal(t.observations[:, 3].cpu().numpy(), oracle.render(blob, lanes, things)["obs"])
    assert np.array_equal(t.observations[:, 2].cpu().numpy(), want)
    e.close()


@pytest.mark.gpu
def test_engine_state_producer_follows_the_engines_decal_rings(pkg, oracle, scenes):
    """An engine that keeps ``hitscan_decal_*`` rings (src/gradoom/engine.py:1870-1884): the producer
    binds them to the renderer and refreshes them with the state, so chips added between two
    steps show up in the next observation."""

    from conftest import fake_engine
    from gradoom_b200 import env as gdenv, state as gdstate, stepper

    sc, blob = scenes("c1d")
    n, slots = 4, 128
    base = fake_engine(n, seed=31)
    lanes, things, _k = oracle.pack_state(blob, base, 64)
    rings = [stepper.random_decals(sc, lanes, count, slots, seed=40 + count) for count in (0, 90)]

    def ring_tensors(engine, rec):
        engine.hitscan_decal_serial = torch.from_numpy(rec[..., 0].copy()).to(DEV)
        engine.hitscan_decal_wall = torch.from_numpy((rec[..., 1] & 0xFFFF).astype(np.int32)).to(DEV)
        engine.hitscan_decal_style = torch.from_numpy((rec[..., 1] >> 16).astype(np.uint8)).to(DEV)
        engine.hitscan_decal_along = torch.from_numpy(rec[..., 2].copy().view(np.float32)).to(DEV)
        engine.hitscan_decal_z = torch.from_numpy(rec[..., 3].copy().view(np.float32)).to(DEV)

    class Engine:
        def __init__(self):
            self.__dict__.update(vars(fake_engine(n, seed=31, device=DEV)))
            self.signal_buffer = torch.zeros((n, 27), device=DEV)
            self.pending_reset = torch.zeros(n, dtype=torch.bool, device=DEV)
            self.render_frame = None
            ring_tensors(self, rings[0])

        def reset(self, mask, seeds):
            self.render_frame(mask)

        def step(self, buttons):
            self.render_frame()
            ring_tensors_in_place(self, rings[1])
            zeros = torch.zeros(n, device=DEV)
            return None, zeros, zeros.bool(), zeros.bool()

    def ring_tensors_in_place(engine, rec):
        fresh = Engine.__new__(Engine)
        ring_tensors(fresh, rec)
        for name in ("serial", "wall", "style", "along", "z"):
            getattr(engine, f"hitscan_decal_{name}").copy_(getattr(fresh, f"hitscan_decal_{name}"))

    engine = Engine()
    assert torch.equal(gdstate.decal_records(engine).cpu(), torch.from_numpy(rings[0]))
    producer = gdenv.EngineStateProducer(engine, sc, 64)
    e = gdenv.GraDoomVecEnv(compiled_scenario=sc, num_envs=n, device=DEV, producer=producer, max_things=64,
                            frame_skip=2, obs_crop=(0, 32, 0, 0), obs_crop_mode="mask")
    obs, _signals = e.reset_device(torch.ones(n, dtype=torch.bool, device=DEV), torch.arange(n, device=DEV))
    bare = oracle.render(blob, lanes, things)["obs"]
    assert np.array_equal(obs[:, 3].cpu().numpy(), bare)
    t = e.step_device(torch.zeros(n, dtype=torch.int64, device=DEV))
    chipped = oracle.render(blob, lanes, things, decals=rings[1].view(oracle.DECAL_DTYPE)[..., 0])["obs"]
    assert not np.array_equal(chipped, bare)
    assert np.array_equal(t.observations[:, 3].cpu().numpy(), chipped)
    e.close()


@pytest.mark.gpu
def test_gym_level_reset_step_and_observation_ownership(pkg, scenes):
    """reset()/step() with the three obs_copy modes (src/gradoom/env.py:678-688; upstream
    tests/test_turbo_api_contract.py:454-465: safe_view alternates two buffers)."""

    n = 4
    actions = torch.full((n,), 2, device=DEV, dtype=torch.int64)
    safe = _env(scenes, n=n, obs_copy="safe_view")
    first, infos = safe.reset(seed=7)
    assert first.shape == (n, 4, 84, 84) and set(("killcount", "_killcount", "state_index")) <= set(infos)
    second = safe.step(actions)[0]
    after_one_step = second.clone()
    third = safe.step(actions)[0]
    assert first.data_ptr() != second.data_ptr() and third.data_ptr() == first.data_ptr()
    assert second.data_ptr() != safe._frames.data_ptr()
    kept = third.clone()
    safe.step(actions)                                   # lands in `second`'s buffer; `third` is still intact
    assert torch.equal(third, kept)
    owned = _env(scenes, n=n, obs_copy="copy")
    a, _ = owned.reset(seed=7)
    b = owned.step(actions)[0]
    assert a.data_ptr() != b.data_ptr() and b.data_ptr() != owned._frames.data_ptr()
    live = _env(scenes, n=n, obs_copy="unsafe_view")
    c, _ = live.reset(seed=7)
    d, rewards, terminated, truncated, info = live.step(actions)
    assert c.data_ptr() == d.data_ptr() == live._frames.data_ptr()
    assert rewards.shape == (n,) and terminated.dtype == torch.bool and "episode_time" in info
    # the same seeds give the same episode in every mode
    assert torch.equal(b, d) and torch.equal(after_one_step, b)
    # masked reset through options, seeds per lane, the asynchronous pair
    mask = torch.tensor([True, False, False, True], device=DEV)
    obs, infos = live.reset(seed=[3, None, None, 9], options={"reset_mask": mask})
    assert torch.equal(infos["_state_index"], mask) and torch.equal(obs[0, 0], obs[0, 3])
    live.step_async(actions)
    with pytest.raises(RuntimeError):
        live.step_async(actions)
    assert live.step_wait()[0].shape == (n, 4, 84, 84)
    with pytest.raises(ValueError):
        live.reset(options={"reset_mask": torch.zeros(n, dtype=torch.bool, device=DEV)})
    with pytest.raises(ValueError):
        live.reset(options={"bogus": 1})
    for e in (safe, owned, live):
        e.close()


@pytest.mark.gpu
def test_constructor_follows_the_reference_keyword_set(pkg, scenes):
    """Names and refusals of src/gradoom/env.py:228-350."""

    from gradoom_b200 import env as gdenv

    sc, _ = scenes("c1")
    base = dict(compiled_scenario=sc, num_envs=2, device=DEV)
    for bad in (dict(players=2), dict(record=True), dict(render_mode="human"), dict(num_threads=4),
                dict(obs_resize=(64, 64)), dict(frame_stack=2), dict(obs_crop=(1, 2, 3, 4)),
                dict(obs_crop=(0, 32, 0, 0), obs_crop_mode="remove"), dict(obs_layout="nhwc"),
                dict(transport="numpy"), dict(obs_copy="view"), dict(observation_renderer="approximate"),
                dict(observation_renderer="bogus"), dict(doom_skill=2), dict(sticky_action_prob=0.25),
                dict(maxpool_last_two=True), dict(vizdoom_config={"fps": 35}), dict(num_envs=0),
                dict(state="other"), dict(doom_map="MAP01"), dict(stack_policy="stack")):
        with pytest.raises(ValueError):
            gdenv.GraDoomVecEnv(**{**base, **bad})
    with pytest.raises(FileNotFoundError):
        gdenv.GraDoomVecEnv(num_envs=2, device=DEV)
    e = gdenv.GraDoomVecEnv("VizdoomDeathmatch-v1", **base)      # the reference's defaults: HUD visible, frame skip 4
    assert e.frame_skip == 4 and e.mask_hud is False and e.obs_copy == "safe_view" and e.observation_renderer == "reference"
    obs, _ = e.reset(seed=1)
    assert obs[:, :, 74:].any()                                   # status-bar rows are drawn when nothing is masked
    e.close()


@pytest.mark.gpu
def test_operator_seam_traces_under_torch_compile(pkg, oracle, scenes):
    """The entry points as torch.library operators (the reference's second plugin
    mechanism, src/gradoom/_triton_kernels.py:180-212): eager and compiled with
    fullgraph=True give the oracle's frames."""

    from gradoom_b200 import native, ops, stepper

    sc, blob = scenes("c1")
    n, k = 6, 4
    r = native.Renderer(blob, DEV, k)
    lanes_np, things_np = stepper.random_lanes(sc, n, k, seed=4)
    expected = oracle.render(blob, lanes_np, things_np)
    lanes, things = torch.from_numpy(lanes_np).to(DEV), torch.from_numpy(things_np).to(DEV)
    handle = r.handle.value
    assert set(ops.NAMES) <= set(dir(torch.ops.gradoom_b200))

    def step(lanes, things, stack, scratch, status):
        torch.ops.gradoom_b200.render_step_(handle, lanes, things, stack, scratch, status, True)
        obs = torch.ops.gradoom_b200.render_observation(handle, lanes, things, scratch, status, True)
        return obs, stack.to(torch.float32).mean()

    stack = torch.zeros((n, 4, 84, 84), dtype=torch.uint8, device=DEV)
    obs, mean = step(lanes, things, stack, r.scratch, r.status)
    assert np.array_equal(obs.cpu().numpy(), expected["obs"]) and np.array_equal(stack[:, 3].cpu().numpy(), expected["obs"])
    compiled = torch.compile(step, fullgraph=True)
    stack2 = torch.zeros_like(stack)
    obs2, mean2 = compiled(lanes, things, stack2, r.scratch, r.status)
    assert torch.equal(obs2, obs) and torch.equal(stack2, stack) and torch.allclose(mean2, mean)
    rgb = torch.ops.gradoom_b200.render_rgb(handle, lanes, things, r.scratch, r.status, True)
    assert np.array_equal(rgb.cpu().numpy(), oracle.rgb(blob, expected["indexed"]))
    r.check_status()
