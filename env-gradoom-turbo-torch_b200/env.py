"""Host-side mirror of the reference's device API for the render path.

``GraDoomVecEnv`` keeps the names, argument meaning, tensor contracts and error
behaviour of the reference's ``GraDoomVecEnv`` for the calls that reach the
renderer (src/gradoom/env.py:851-942, 998-1066):

* ``reset_device(mask, seeds) -> (observations, signals)``
* ``step_device(actions) -> DeviceTransition``
* ``step_and_reset_device(actions, reset_seeds) -> DeviceAutoResetTransition``
* ``render() / render_lane(lane) / get_images()`` -- 240x320x3 RGB24 numpy
* ``device_signals()``, ``close()``

Game dynamics are not part of this package: the environment drives a *state
producer* -- any object with ``reset(mask, seeds)`` and ``step(buttons) ->
(rewards, terminated, truncated)`` that can hand over packed lane / thing
records (``render_inputs()``) and a ``signal_buffer``.  ``stepper.LaneStepper``
is the built-in producer for throughput runs; ``EngineStateProducer`` adapts an
object carrying the reference engine's tensors.  Every frame is drawn by the
CUDA library; there is no other renderer behind this class.
"""

from __future__ import annotations

import operator
from dataclasses import dataclass

import numpy as np
import torch

from . import native
from . import scene as gdscene
from . import state as gdstate

# Pinned buttons and the 17 pinned actions (src/gradoom/actions.py:10-51).
DEATHMATCH_BUTTONS = (
    "ATTACK", "SPEED", "STRAFE", "MOVE_RIGHT", "MOVE_LEFT", "MOVE_BACKWARD", "MOVE_FORWARD", "TURN_RIGHT",
    "TURN_LEFT", "SELECT_WEAPON1", "SELECT_WEAPON2", "SELECT_WEAPON3", "SELECT_WEAPON4", "SELECT_WEAPON5",
    "SELECT_WEAPON6", "SELECT_NEXT_WEAPON", "SELECT_PREV_WEAPON", "LOOK_UP_DOWN_DELTA",
    "TURN_LEFT_RIGHT_DELTA", "MOVE_LEFT_RIGHT_DELTA",
)
DEATHMATCH_ACTIONS = (
    (), ("ATTACK",), ("MOVE_FORWARD",), ("MOVE_BACKWARD",), ("MOVE_LEFT",), ("MOVE_RIGHT",), ("TURN_LEFT",),
    ("TURN_RIGHT",), ("SPEED", "MOVE_FORWARD"), ("ATTACK", "MOVE_FORWARD"), ("ATTACK", "MOVE_BACKWARD"),
    ("ATTACK", "MOVE_LEFT"), ("ATTACK", "MOVE_RIGHT"), ("ATTACK", "TURN_LEFT"), ("ATTACK", "TURN_RIGHT"),
    ("SELECT_NEXT_WEAPON",), ("SELECT_PREV_WEAPON",),
)
_ACTION_DTYPES = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
# columns of the signal buffer (src/gradoom/engine.py:509-539)
DEVICE_SIGNAL_NAMES = (
    "killcount", "health", "armor", "selected_weapon", "selected_weapon_ammo", "weapon1", "weapon2", "weapon3",
    "weapon4", "weapon5", "weapon6", "ammo1", "ammo2", "ammo3", "ammo4", "ammo5", "ammo6", "episode_time",
    "episode_return", "player_dead", "pending_reset", "deathcount", "hitcount", "damagecount", "hits_taken",
    "damage_taken", "player_killcount",
)


def _normalize_seed(seed, num_envs: int):
    """One seed per lane from None, an int (lane i gets seed + i) or a sequence
    (src/gradoom/env.py:101-113)."""

    if seed is None:
        return [None] * num_envs
    if isinstance(seed, (list, tuple, np.ndarray)):
        result = [None if value is None else int(value) for value in seed]
        if len(result) != num_envs:
            raise ValueError("seed sequence length must match num_envs")
        return result
    return [int(seed) + lane for lane in range(num_envs)]


@dataclass(frozen=True)
class DeviceTransition:
    observations: torch.Tensor
    rewards: torch.Tensor
    terminated: torch.Tensor
    truncated: torch.Tensor
    signals: torch.Tensor
    info_histories: torch.Tensor


@dataclass(frozen=True)
class DeviceAutoResetTransition:
    observations: torch.Tensor
    rewards: torch.Tensor
    terminated: torch.Tensor
    truncated: torch.Tensor
    signals: torch.Tensor
    info_histories: torch.Tensor
    final_observations: torch.Tensor
    final_signals: torch.Tensor
    final_info_histories: torch.Tensor


def action_matrix(device) -> torch.Tensor:
    m = torch.zeros((len(DEATHMATCH_ACTIONS), len(DEATHMATCH_BUTTONS)), dtype=torch.bool)
    for i, labels in enumerate(DEATHMATCH_ACTIONS):
        for label in labels:
            m[i, DEATHMATCH_BUTTONS.index(label)] = True
    return m.to(device)


def require_device_tensor(value, name, *, device, shape, dtypes) -> torch.Tensor:
    """Boundary validation with the reference's exception types
    (src/gradoom/env.py:711-728)."""

    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a Torch tensor")
    if value.device != device:
        raise TypeError(f"{name} must be on device {device}")
    if tuple(value.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}")
    if value.dtype not in dtypes:
        expected = ", ".join(str(d) for d in dtypes)
        raise TypeError(f"{name} must have dtype {expected}")
    return value


def check_lane_index(lane, num_envs: int) -> int:
    """Lane argument of render_lane (src/gradoom/env.py:1038-1044)."""

    if isinstance(lane, (bool, np.bool_)):
        raise TypeError("lane must be an integer")
    index = operator.index(lane)
    if not 0 <= index < num_envs:
        raise IndexError(f"lane must be in [0, {num_envs - 1}]")
    return index


class EngineStateProducer:
    """Adapts an object with the reference engine's lane tensors and methods
    (``reset``, ``step``, ``signal_buffer``; src/gradoom/engine.py:2261, 9550)
    to the producer protocol, packing its state for the renderer each call."""

    def __init__(self, engine, sc: gdscene.Scene, max_things: int):
        self.engine = engine
        self.state = gdstate.EngineState(engine)
        self.max_things = max_things
        self.num_envs = engine.x.shape[0]
        self.renderer = None            # bound by the environment once it owns one
        self._lanes = self._things = None

    @property
    def signal_buffer(self):
        return self.engine.signal_buffer

    @property
    def pending_reset(self):
        return self.engine.pending_reset

    def reset(self, mask, seeds):
        render_frame = self.engine.render_frame
        self.engine.render_frame = lambda active=None: torch.zeros(
            (self.num_envs, 84, 84), dtype=torch.uint8, device=self.engine.x.device)
        try:
            self.engine.reset(mask, seeds)
        finally:
            self.engine.render_frame = render_frame

    def step(self, buttons):
        render_frame = self.engine.render_frame
        self.engine.render_frame = lambda active=None: torch.zeros(
            (self.num_envs, 84, 84), dtype=torch.uint8, device=self.engine.x.device)
        try:
            _frames, rewards, terminated, truncated = self.engine.step(buttons)
        finally:
            self.engine.render_frame = render_frame
        return rewards, terminated, truncated

    def bind_renderer(self, renderer):
        self.renderer = renderer
        dev = renderer.device
        self._lanes = torch.zeros((self.num_envs, gdstate.LANE_WORDS), dtype=torch.int32, device=dev)
        self._things = torch.zeros((self.num_envs, max(self.max_things, 1), 4), dtype=torch.int32, device=dev)
        # the engine's bullet-chip rings (src/gradoom/engine.py:1870-1884), when it keeps any
        self._decals = None
        if hasattr(self.engine, "hitscan_decal_serial"):
            self._decals = gdstate.decal_records(self.engine).to(dev).contiguous()
            renderer.bind_decals(self._decals)

    def render_inputs(self):
        """Lane and thing records of the engine's present state, packed on the
        device by the library (gd_pack_state)."""

        if self.renderer is None:
            raise RuntimeError("bind_renderer() must be called before render_inputs()")
        self.renderer.pack_state(self.state.refresh(), self._lanes, self._things)
        if self._decals is not None:
            gdstate.decal_records(self.engine, out=self._decals)
        return self._lanes, self._things


class GraDoomVecEnv:
    """Device-resident vector environment whose observations come from the CUDA renderer."""

    metadata = {
        "render_modes": ["rgb_array"],
        "render_fps": 35,
        "turbo_api_version": 2,
        "transition_transport": "torch",
        "gradoom_device_api_version": 1,
    }

    def __init__(self, game=None, state=None, scenario=None, info=None, use_restricted_actions="default",
                 record: bool = False, players: int = 1, inttype="stable", obs_type="image",
                 render_mode: str | None = None, *, num_envs: int = 1, num_threads: int | None = None,
                 rom_path: str | None = None, transport: str = "default", obs_copy: str = "safe_view",
                 obs_resize=(84, 84), obs_crop=None, obs_crop_mode: str = "remove", obs_crop_fill: int = 0,
                 obs_grayscale: bool = True, obs_resize_algorithm: str = "area", obs_layout: str = "chw",
                 frame_skip: int = 4, frame_stack: int = 4, maxpool_last_two: bool = False,
                 noop_reset_max: int = 0, use_fire_reset: bool = False, sticky_action_prob: float = 0.0,
                 reward_clip=False, info_filter="all", info_frame_stack_keys=None, state_catalog=None,
                 device=None, doom_map=None, doom_skill=None, wall_contact_damage_scale: float = 1.0,
                 observation_renderer: str = "reference", game_args=None, game_variables=None,
                 enemy_variants=None, surface_variants=None, treat_episode_timeout_as_truncation: bool = True,
                 vizdoom_config=None, compiled_scenario=None, require_pinned_scenario: bool = True,
                 compile_engine: bool = False,
                 # beyond the reference's keyword set: the state producer and the renderer's options
                 producer=None, max_things: int = 16, producer_seed: int = 0, stack_policy: str = "roll"):
        """Keyword-compatible with the reference's constructor (src/gradoom/env.py:228-350): the
        same names, defaults and refusals for what the deathmatch profile does not support.
        Differences, all refusals or additions: the scene must be handed over compiled
        (``compiled_scenario=``: a ``scene.Scene`` of this package, or the reference's
        ``CompiledScenario``; WAD compilation is not part of this library);
        ``observation_renderer`` must be ``"reference"`` -- the native pipeline is the one
        renderer behind this class, and it is also the default here; ``info_frame_stack_keys``
        is not supported."""

        if transport == "default":
            transport = "torch"
        if info not in (None, "data"):
            raise ValueError("info must be None or 'data'")
        if record:
            raise ValueError("record=True is not supported on the device path")
        if players != 1:
            raise ValueError("the deathmatch-p1-v1 profile supports players=1")
        if str(obs_type).split(".")[-1].casefold() != "image":
            raise ValueError("GraDoomVecEnv supports image observations only")
        if render_mode not in (None, "rgb_array"):
            raise ValueError("render_mode must be None or 'rgb_array'")
        if state is not None and state_catalog is not None:
            raise ValueError("state and state_catalog are mutually exclusive")
        catalog = ("default",) if state_catalog is None else tuple(state_catalog)
        if state not in (None, "default") or catalog != ("default",):
            raise ValueError("the first device profile supports only the default initial state")
        if any(value is not None for value in (doom_map, game_args, enemy_variants, surface_variants)):
            raise ValueError("custom maps, game args, and variants are not yet supported")
        if doom_skill not in (None, 1, 3):
            raise ValueError("deathmatch-p1-v1 supports Doom skill 1 or 3")
        if observation_renderer not in ("approximate", "native-fused", "reference"):
            raise ValueError("observation_renderer must be 'approximate', 'native-fused', or 'reference'")
        if observation_renderer != "reference":
            raise ValueError("this library draws observation_renderer='reference' (the native pipeline) only")
        if use_fire_reset or noop_reset_max or sticky_action_prob:
            raise ValueError("fire reset, no-op reset, and sticky actions are not in deathmatch-p1-v1")
        if maxpool_last_two:
            raise ValueError("deathmatch-p1-v1 does not max-pool consecutive frames")
        if tuple(obs_resize or ()) != (84, 84) or not obs_grayscale or frame_stack != 4:
            raise ValueError("deathmatch-p1-v1 requires 84x84 grayscale frame-stack 4")
        if obs_crop is not None:
            obs_crop = tuple(obs_crop)
        if obs_crop not in (None, (0, 32, 0, 0)):
            raise ValueError("deathmatch-p1-v1 supports no crop or the pinned bottom-32 mask")
        if obs_crop is not None and (obs_crop_mode != "mask" or obs_crop_fill != 0):
            raise ValueError("the pinned deathmatch crop is a zero-filled mask")
        if obs_crop is None and obs_crop_mode not in ("remove", "mask"):
            raise ValueError("obs_crop_mode must be 'remove' or 'mask'")
        if obs_crop_fill != 0:
            raise ValueError("deathmatch-p1-v1 requires obs_crop_fill=0")
        if obs_layout not in ("chw", "hwc"):
            raise ValueError("obs_layout must be 'chw' or 'hwc'")
        if obs_resize_algorithm != "area":
            raise ValueError("deathmatch-p1-v1 supports obs_resize_algorithm='area' only")
        if transport != "torch":
            raise ValueError("transport must be 'torch'; NumPy transition transport is unsupported")
        if obs_copy not in ("copy", "safe_view", "unsafe_view"):
            raise ValueError("obs_copy must be copy, safe_view, or unsafe_view")
        if str(getattr(inttype, "name", inttype)).split(".")[-1].casefold() != "stable":
            raise ValueError("inttype must select the Stable integration")
        if num_threads is not None:
            raise ValueError("num_threads is unsupported and must be None on the device path")
        if isinstance(num_envs, bool) or not isinstance(num_envs, (int, np.integer)) or num_envs <= 0:
            raise ValueError("num_envs must be a positive integer")
        if isinstance(frame_skip, bool) or not isinstance(frame_skip, (int, np.integer)) or frame_skip <= 0:
            raise ValueError("frame_skip must be a positive integer")
        if info_frame_stack_keys:
            raise ValueError("info_frame_stack_keys are not supported by this library")
        if not treat_episode_timeout_as_truncation:
            raise ValueError("deathmatch-p1-v1 treats its native timeout as truncation")
        if stack_policy not in ("roll", "ring"):
            raise ValueError("stack_policy must be 'roll' or 'ring'")
        options = dict(vizdoom_config or {})
        unknown = set(options) - {"episode_timeout", "render_screen_flashes"}
        if unknown:
            raise ValueError(f"unsupported vizdoom_config keys: {sorted(unknown)}")
        episode_timeout = options.get("episode_timeout", 4200)
        if isinstance(episode_timeout, bool) or not isinstance(episode_timeout, (int, np.integer)) or episode_timeout <= 0:
            raise ValueError("episode_timeout must be a positive integer")
        self.render_screen_flashes = options.get("render_screen_flashes", False)
        if not isinstance(self.render_screen_flashes, bool):
            raise ValueError("render_screen_flashes must be a boolean")
        if compiled_scenario is None:
            raise FileNotFoundError("pass compiled_scenario=...: this library does not compile WAD files")
        sc = compiled_scenario if isinstance(compiled_scenario, gdscene.Scene) \
            else gdscene.from_compiled_scenario(compiled_scenario)
        if device is None:
            device = "cuda"
        self.game = str(game or "VizdoomDeathmatch-v1")
        self.obs_copy = obs_copy
        self.observation_renderer = observation_renderer
        self.transport = transport
        self.compiled_scenario = compiled_scenario
        self._safe_obs_index = 0
        self._pending_actions = None
        self._seed_values = [None] * int(num_envs)
        self._reset_rngs = [np.random.default_rng(lane) for lane in range(int(num_envs))]
        self._reward_clip = self._normalize_reward_clip(reward_clip)
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.num_envs = int(num_envs)
        self.frame_skip = int(frame_skip)
        self.frame_stack = 4
        self.render_mode = render_mode
        self.obs_layout = obs_layout
        self.mask_hud = obs_crop is not None
        self.scene = sc
        self.closed = False
        blob = gdscene.pack_scene(sc)
        self._renderer = native.Renderer(blob, self.device, max_things)
        if producer is None:
            from .stepper import LaneStepper

            producer = LaneStepper(sc, self.num_envs, device=self.device, k_things=min(max_things, 12),
                                   max_things=max_things, frame_skip=frame_skip, episode_timeout=episode_timeout,
                                   seed=producer_seed)
        self._producer = producer
        if hasattr(producer, "bind_renderer"):
            producer.bind_renderer(self._renderer)
        # "roll": the reference's contiguous oldest-first stack, shifted every step.  "ring": eight
        # slots per lane written twice and never moved; observations are then a strided (N,4,84,84)
        # view of the same four frames (valid until the next step, like the reference's).
        self.stack_policy = stack_policy
        self._ring_head = 3
        slots = 4 if stack_policy == "roll" else 8
        self._frames = torch.zeros((self.num_envs, slots, 84, 84), dtype=torch.uint8, device=self.device)
        self._initialized = torch.zeros(self.num_envs, dtype=torch.bool, device=self.device)
        self._action_matrix = action_matrix(self.device)
        shape = (4, 84, 84) if obs_layout == "chw" else (84, 84, 4)
        self._safe_obs_buffers = tuple(torch.empty((self.num_envs, *shape), dtype=torch.uint8, device=self.device)
                                       for _ in range(2)) if obs_copy == "safe_view" else ()
        self._info_history = torch.zeros((self.num_envs, 0, 4), dtype=torch.float32, device=self.device)
        self._state_indices = torch.zeros(self.num_envs, dtype=torch.int32, device=self.device)
        self.action_table = DEATHMATCH_ACTIONS
        self.buttons = DEATHMATCH_BUTTONS

    # -- helpers ---------------------------------------------------------
    def _device_observations(self) -> torch.Tensor:
        frames = self._frames
        if self.stack_policy == "ring":
            frames = frames[:, self._ring_head + 1:self._ring_head + 5]
        return frames if self.obs_layout == "chw" else frames.permute(0, 2, 3, 1)

    def _require_open(self, what: str) -> None:
        if self.closed:
            raise RuntimeError(f"cannot {what} a closed environment")

    # -- device API ------------------------------------------------------
    def reset_device(self, mask: torch.Tensor, seeds: torch.Tensor):
        self._require_open("reset")
        mask = require_device_tensor(mask, "mask", device=self.device, shape=(self.num_envs,), dtypes=(torch.bool,))
        seeds = require_device_tensor(seeds, "seeds", device=self.device, shape=(self.num_envs,),
                                      dtypes=_ACTION_DTYPES).to(torch.int64)
        self._producer.reset(mask, seeds)
        lanes, things = self._producer.render_inputs()
        if self.stack_policy == "ring":
            self._renderer.reset_ring(lanes, things, mask, self._frames, mask_hud=self.mask_hud)
        else:
            self._renderer.reset(lanes, things, mask, self._frames, mask_hud=self.mask_hud)
        self._initialized |= mask
        return self._device_observations(), self._producer.signal_buffer

    def step_device(self, actions: torch.Tensor) -> DeviceTransition:
        self._require_open("step")
        indices = require_device_tensor(actions, "actions", device=self.device, shape=(self.num_envs,),
                                        dtypes=_ACTION_DTYPES).to(torch.int64)
        buttons = self._action_matrix[indices]
        rewards, terminated, truncated = self._producer.step(buttons)
        lanes, things = self._producer.render_inputs()
        if self.stack_policy == "ring":
            self._ring_head = (self._ring_head + 1) & 3
            self._renderer.step_ring(lanes, things, self._frames, self._ring_head, mask_hud=self.mask_hud)
        else:
            self._renderer.step(lanes, things, self._frames, mask_hud=self.mask_hud)
        return DeviceTransition(self._device_observations(), rewards, terminated, truncated,
                                self._producer.signal_buffer, self._info_history)

    @staticmethod
    def _normalize_reward_clip(value):
        if value is False:
            return None
        if value is True:
            return (-1.0, 1.0)
        try:
            low, high = (float(item) for item in value)
        except (TypeError, ValueError) as exc:
            raise ValueError("reward_clip must be a bool or a (low, high) pair") from exc
        if not np.isfinite(low) or not np.isfinite(high) or low > high:
            raise ValueError("reward_clip bounds must be finite with low <= high")
        return low, high

    # -- gym-level API (src/gradoom/env.py:678-688, 746-848) ------------------
    def _observations(self, values: torch.Tensor) -> torch.Tensor:
        """Ownership of the observations a gym-level call returns: ``copy`` clones, ``safe_view``
        alternates two buffers (a returned tensor stays intact for one more call), ``unsafe_view``
        hands out the live stack."""

        if self.obs_copy == "copy":
            return values.clone()
        if self.obs_copy == "safe_view":
            buffer = self._safe_obs_buffers[self._safe_obs_index]
            self._safe_obs_index = (self._safe_obs_index + 1) % len(self._safe_obs_buffers)
            buffer.copy_(values)
            return buffer
        return values

    def _infos(self, availability=None) -> dict:
        if availability is None:
            availability = torch.ones(self.num_envs, dtype=torch.bool, device=self.device)
        signals = self._producer.signal_buffer
        result = {}
        for index, name in enumerate(DEVICE_SIGNAL_NAMES):
            result[name] = signals[:, index].to(torch.float64)
            result[f"_{name}"] = availability.clone()
        return result

    def seed(self, seed=None):
        self._seed_values = _normalize_seed(seed, self.num_envs)
        return list(self._seed_values)

    def reset(self, *, seed=None, options=None):
        self._require_open("reset")
        reset_options = dict(options or {})
        raw_mask = reset_options.pop("reset_mask", None)
        if raw_mask is None:
            mask = torch.ones(self.num_envs, dtype=torch.bool, device=self.device)
        else:
            mask = require_device_tensor(raw_mask, "options['reset_mask']", device=self.device,
                                         shape=(self.num_envs,), dtypes=(torch.bool,))
        if not bool(torch.any(mask)):
            raise ValueError("options['reset_mask'] must select at least one lane")
        state_indices = reset_options.pop("state_indices", None)
        if state_indices is not None:
            selected = require_device_tensor(state_indices, "options['state_indices']", device=self.device,
                                             shape=(self.num_envs,), dtypes=(torch.int32,))
            if bool(torch.any(selected[mask] != 0)):
                raise ValueError("deathmatch-p1-v1 has only state index 0")
        if reset_options:
            raise ValueError(f"unsupported reset options: {sorted(reset_options)}")
        seed_values = _normalize_seed(seed, self.num_envs) if seed is not None else self._seed_values
        game_seeds = [0] * self.num_envs
        for lane in torch.nonzero(mask, as_tuple=False).flatten().to("cpu").tolist():
            if seed_values[lane] is not None:
                self._reset_rngs[lane] = np.random.default_rng(seed_values[lane])
            game_seeds[lane] = int(self._reset_rngs[lane].integers(0, np.iinfo(np.uint32).max + 1, dtype=np.uint32))
        self._seed_values = [None] * self.num_envs
        observations, _signals = self.reset_device(mask, torch.tensor(game_seeds, dtype=torch.int64, device=self.device))
        infos = self._infos(mask)
        infos["state_index"] = self._state_indices.clone()
        infos["_state_index"] = mask.clone()
        return self._observations(observations), infos

    def step(self, actions: torch.Tensor):
        """Validated step (host synchronising, like the reference's gym ``step``)."""

        self._require_open("step")
        if not bool(torch.all(self._initialized)):
            raise RuntimeError("all lanes must be reset before the first step")
        pending = self._producer.pending_reset
        if bool(torch.any(pending)):
            lanes = torch.nonzero(pending).flatten().to("cpu").tolist()
            raise RuntimeError(f"terminal lanes must be reset before step: {lanes}")
        indices = require_device_tensor(actions, "actions", device=self.device, shape=(self.num_envs,),
                                        dtypes=_ACTION_DTYPES).to(torch.int64)
        if bool(torch.any((indices < 0) | (indices >= len(self.action_table)))):
            raise ValueError("actions fall outside the declared action space")
        t = self.step_device(indices)
        rewards = t.rewards if self._reward_clip is None else t.rewards.clamp(*self._reward_clip)
        return self._observations(t.observations), rewards, t.terminated, t.truncated, self._infos()

    def step_async(self, actions: torch.Tensor) -> None:
        if self._pending_actions is not None:
            raise RuntimeError("an asynchronous step is already pending")
        self._pending_actions = actions

    def step_wait(self):
        if self._pending_actions is None:
            raise RuntimeError("no asynchronous step is pending")
        actions, self._pending_actions = self._pending_actions, None
        return self.step(actions)

    def step_and_reset_device(self, actions: torch.Tensor, reset_seeds: torch.Tensor) -> DeviceAutoResetTransition:
        t = self.step_device(actions)
        final_observations = t.observations.clone()
        final_signals = t.signals.clone()
        final_info = t.info_histories.clone()
        done = t.terminated | t.truncated
        # Unlike the reference (src/gradoom/env.py:919) no host sync decides whether
        # to reset: the reset kernel skips unmasked lanes on the device.
        observations, signals = self.reset_device(done, reset_seeds)
        return DeviceAutoResetTransition(observations, t.rewards, t.terminated, t.truncated, signals,
                                         self._info_history, final_observations, final_signals, final_info)

    def device_signals(self) -> torch.Tensor:
        return self._producer.signal_buffer

    def device_info_histories(self) -> torch.Tensor:
        return self._info_history

    def active_state_indices(self) -> torch.Tensor:
        """Index of the scenario state every lane runs (src/gradoom/env.py:392-394, 1034): one
        scenario, so all zeros."""

        return self._state_indices

    # -- diagnostic RGB --------------------------------------------------
    def _render_rgb(self, first: int, count: int) -> np.ndarray:
        lanes, things = self._producer.render_inputs()
        lanes = lanes[first:first + count].contiguous()
        things = things[first:first + count].contiguous()
        _, _, rgb = self._renderer.frames(lanes, things, rgb=True, mask_hud=self.mask_hud, include_hud=True)
        return rgb.to("cpu").numpy()

    def render_lane(self, lane: int):
        self._require_open("render")
        index = check_lane_index(lane, self.num_envs)
        if self.render_mode != "rgb_array":
            return None
        return self._render_rgb(index, 1)[0].copy()

    def render(self):
        return self.render_lane(0)

    def get_images(self):
        self._require_open("render")
        if self.render_mode != "rgb_array":
            return [None for _ in range(self.num_envs)]
        return [frame.copy() for frame in self._render_rgb(0, self.num_envs)]

    def check_status(self) -> None:
        self._renderer.check_status()

    def close(self) -> None:
        if not self.closed:
            self._renderer.close()
        self.closed = True
