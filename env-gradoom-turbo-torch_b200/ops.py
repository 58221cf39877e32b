"""The render entry points as ``torch.library`` operators.

The reference reaches its device kernels through a second seam besides the
renderer callable: every kernel is a ``torch.library.custom_op`` with a fake
implementation, so that code built on them traces under ``torch.compile``
(src/gradoom/_triton_kernels.py:180-212; the name list and the raising stubs for a
missing backend: src/gradoom/_kernels.py:8-65).  This module gives the C ABI of this
library the same shape: ``torch.ops.gradoom_b200.<name>``; operators that work in
place end in ``_`` and return nothing; each has a fake for tracing; a missing
shared library makes every call raise (``native.NativeError``, a ``RuntimeError``).
``renderer`` is the integer value of a ``gd_renderer*`` (``native.Renderer.handle.value``).
"""

from __future__ import annotations

import torch

from . import native

NAMESPACE = "gradoom_b200"
NAMES = ("render_step_", "render_reset_", "render_observation", "render_rgb", "player_tics_")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(code: int, what: str) -> None:
    if code != native.GD_OK:
        raise native.NativeError(f"{what} failed: {native.load().gd_error_string(code).decode()} ({code})")


@torch.library.custom_op(f"{NAMESPACE}::render_step_", mutates_args=("stack", "scratch", "status"), device_types="cuda")
def render_step_(renderer: int, lanes: torch.Tensor, things: torch.Tensor, stack: torch.Tensor, scratch: torch.Tensor,
                 status: torch.Tensor, mask_hud: bool) -> None:
    """gd_render_step: draw every lane and push the frame onto ``stack (N,4,84,84)``."""

    with torch.cuda.device(lanes.device):
        _check(native.load().gd_render_step(renderer, lanes.data_ptr(), things.data_ptr(), lanes.shape[0], int(mask_hud),
                                            stack.data_ptr(), scratch.data_ptr(), scratch.numel(), status.data_ptr(),
                                            _stream(lanes)), "gd_render_step")


@render_step_.register_fake
def _(renderer, lanes, things, stack, scratch, status, mask_hud):
    return None


@torch.library.custom_op(f"{NAMESPACE}::render_reset_", mutates_args=("stack", "scratch", "status"), device_types="cuda")
def render_reset_(renderer: int, lanes: torch.Tensor, things: torch.Tensor, reset_mask: torch.Tensor, stack: torch.Tensor,
                  scratch: torch.Tensor, status: torch.Tensor, mask_hud: bool) -> None:
    """gd_render_reset: fill all four slots of the lanes whose ``reset_mask`` byte is set."""

    with torch.cuda.device(lanes.device):
        _check(native.load().gd_render_reset(renderer, lanes.data_ptr(), things.data_ptr(), lanes.shape[0], int(mask_hud),
                                             reset_mask.data_ptr(), stack.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                             status.data_ptr(), _stream(lanes)), "gd_render_reset")


@render_reset_.register_fake
def _(renderer, lanes, things, reset_mask, stack, scratch, status, mask_hud):
    return None


@torch.library.custom_op(f"{NAMESPACE}::render_observation", mutates_args=("scratch", "status"), device_types="cuda")
def render_observation(renderer: int, lanes: torch.Tensor, things: torch.Tensor, scratch: torch.Tensor,
                       status: torch.Tensor, mask_hud: bool) -> torch.Tensor:
    """gd_render_frames, observation only: ``(N,84,84) uint8`` (the reference's ``render_frame``)."""

    out = torch.empty((lanes.shape[0], 84, 84), dtype=torch.uint8, device=lanes.device)
    with torch.cuda.device(lanes.device):
        _check(native.load().gd_render_frames(renderer, lanes.data_ptr(), things.data_ptr(), lanes.shape[0], int(mask_hud),
                                              0, out.data_ptr(), None, None, scratch.data_ptr(), scratch.numel(),
                                              status.data_ptr(), _stream(lanes)), "gd_render_frames")
    return out


@render_observation.register_fake
def _(renderer, lanes, things, scratch, status, mask_hud):
    return lanes.new_empty((lanes.shape[0], 84, 84), dtype=torch.uint8)


@torch.library.custom_op(f"{NAMESPACE}::render_rgb", mutates_args=("scratch", "status"), device_types="cuda")
def render_rgb(renderer: int, lanes: torch.Tensor, things: torch.Tensor, scratch: torch.Tensor, status: torch.Tensor,
               include_hud: bool) -> torch.Tensor:
    """gd_render_frames, RGB24 only: ``(N,240,320,3) uint8`` (the reference's ``render_native_frame``)."""

    out = torch.empty((lanes.shape[0], 240, 320, 3), dtype=torch.uint8, device=lanes.device)
    with torch.cuda.device(lanes.device):
        _check(native.load().gd_render_frames(renderer, lanes.data_ptr(), things.data_ptr(), lanes.shape[0], 1,
                                              int(include_hud), None, None, out.data_ptr(), scratch.data_ptr(),
                                              scratch.numel(), status.data_ptr(), _stream(lanes)), "gd_render_frames")
    return out


@render_rgb.register_fake
def _(renderer, lanes, things, scratch, status, include_hud):
    return lanes.new_empty((lanes.shape[0], 240, 320, 3), dtype=torch.uint8)


@torch.library.custom_op(f"{NAMESPACE}::player_tics_", mutates_args=("players", "lanes", "status"), device_types="cuda")
def player_tics_(renderer: int, players: torch.Tensor, buttons: torch.Tensor, lanes: torch.Tensor, status: torch.Tensor,
                 tics: int, episode_timeout: int) -> None:
    """gd_player_tics without solid actors: advance the player records and refresh the lane records."""

    with torch.cuda.device(players.device):
        _check(native.load().gd_player_tics(renderer, players.data_ptr(), buttons.data_ptr(), None, players.shape[0],
                                            tics, episode_timeout, lanes.data_ptr(), status.data_ptr(),
                                            _stream(players)), "gd_player_tics")


@player_tics_.register_fake
def _(renderer, players, buttons, lanes, status, tics, episode_timeout):
    return None
