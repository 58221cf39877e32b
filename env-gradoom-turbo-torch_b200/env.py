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

    def render_inputs(self):
        """Lane and thing records of the engine's present state, packed on the
        device by the library (gd_pack_state)."""

        if self.renderer is None:
            raise RuntimeError("bind_renderer() must be called before render_inputs()")
        self.renderer.pack_state(self.state.refresh(), self._lanes, self._things)
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

    def __init__(self, sc: gdscene.Scene, num_envs: int, *, device, producer=None, max_things: int = 16,
                 frame_skip: int = 2, render_mode: str | None = None, obs_crop=(0, 32, 0, 0),
                 obs_crop_mode: str = "mask", obs_layout: str = "chw", episode_timeout: int = 4200,
                 producer_seed: int = 0, stack_policy: str = "roll"):
        if num_envs <= 0:
            raise ValueError("num_envs must be positive")
        if render_mode not in (None, "rgb_array"):
            raise ValueError("render_mode must be None or 'rgb_array'")
        if obs_layout not in ("chw", "hwc"):
            raise ValueError("obs_layout must be 'chw' or 'hwc'")
        if stack_policy not in ("roll", "ring"):
            raise ValueError("stack_policy must be 'roll' or 'ring'")
        if obs_crop not in (None, (0, 32, 0, 0)) or (obs_crop is not None and obs_crop_mode != "mask"):
            raise ValueError("only obs_crop=None or obs_crop=(0, 32, 0, 0) with obs_crop_mode='mask' is supported")
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
        return t.observations, t.rewards, t.terminated, t.truncated, {}

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
