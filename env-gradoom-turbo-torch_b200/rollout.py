"""Rollout loop around the environment: the trainer-shaped caller of the render path.

Mirrors, in shape, the pieces the reference's learner wraps around
``step_and_reset_device`` (train.py: the kill-count delta reward 1221-1253, the
rollout buffer with its generalised advantage estimate 1524-1672, acting under bf16
autocast 1500-1521 and the collection loop 2888-2901), for the rollout workload of
the benchmark definition: a Nature-CNN (conv32 8x8/4, conv64 4x4/2, conv64 3x3/1,
FC512, 17 logits + 1 value) picks the actions, +1 per kill, GAE(gamma, lambda), one
clipped policy-gradient pass per rollout.  The policy is plain PyTorch: it is the
context the render path runs in, not part of it.  Everything stays on the device; a
whole rollout can be captured in a CUDA graph because the environment's calls
allocate nothing and never synchronise.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .env import DEVICE_SIGNAL_NAMES


class KillcountReward:
    """+1 for every increment of a kill signal between two steps of a lane; the
    counter starts over when the lane's episode ends."""

    def __init__(self, num_envs: int, device, signal_name: str = "killcount"):
        if signal_name not in DEVICE_SIGNAL_NAMES:
            raise ValueError(f"kill reward signals are missing: [{signal_name!r}]")
        self.column = DEVICE_SIGNAL_NAMES.index(signal_name)
        self.previous = torch.zeros(num_envs, dtype=torch.float32, device=device)

    def __call__(self, final_signals, terminated, truncated):
        kills = final_signals[:, self.column]
        reward = (kills - self.previous).clamp_min(0.0)
        self.previous.copy_(torch.where(terminated | truncated, torch.zeros_like(kills), kills))
        return reward


class RolloutStore:
    """Preallocated (steps, lanes, ...) tensors of one rollout and its advantage estimate."""

    def __init__(self, n_steps: int, n_envs: int, device):
        batch = (n_steps, n_envs)
        self.observations = torch.empty((*batch, 4, 84, 84), dtype=torch.uint8, device=device)
        self.actions = torch.empty(batch, dtype=torch.int64, device=device)
        self.rewards = torch.empty(batch, dtype=torch.float32, device=device)
        self.values = torch.empty(batch, dtype=torch.float32, device=device)
        self.log_probs = torch.empty(batch, dtype=torch.float32, device=device)
        self.episode_starts = torch.empty(batch, dtype=torch.bool, device=device)
        self.advantages = torch.empty(batch, dtype=torch.float32, device=device)
        self.returns = torch.empty(batch, dtype=torch.float32, device=device)
        self.n_steps, self.n_envs = n_steps, n_envs

    def add(self, step, observations, episode_starts, actions, rewards, values, log_probs):
        self.observations[step].copy_(observations)
        self.episode_starts[step].copy_(episode_starts)
        self.actions[step].copy_(actions)
        self.rewards[step].copy_(rewards)
        self.values[step].copy_(values)
        self.log_probs[step].copy_(log_probs)

    def finish(self, last_values, dones, gamma: float, gae_lambda: float):
        """Generalised advantage estimate, bootstrapping from ``last_values`` unless the last
        step ended the episode; a step whose successor starts an episode does not bootstrap."""

        running = torch.zeros(self.n_envs, dtype=torch.float32, device=self.rewards.device)
        for step in reversed(range(self.n_steps)):
            if step == self.n_steps - 1:
                alive, following = (~dones).float(), last_values.float()
            else:
                alive, following = (~self.episode_starts[step + 1]).float(), self.values[step + 1]
            delta = self.rewards[step] + gamma * following * alive - self.values[step]
            running = delta + gamma * gae_lambda * alive * running
            self.advantages[step].copy_(running)
        self.returns.copy_(self.advantages + self.values)


class NatureCnnPolicy(nn.Module):
    """conv32 8x8/4 -> conv64 4x4/2 -> conv64 3x3/1 -> FC512 -> action logits + value."""

    def __init__(self, actions: int = 17):
        super().__init__()
        self.trunk = nn.Sequential(
            nn.Conv2d(4, 32, 8, 4), nn.ReLU(), nn.Conv2d(32, 64, 4, 2), nn.ReLU(), nn.Conv2d(64, 64, 3, 1), nn.ReLU(),
            nn.Flatten(), nn.Linear(64 * 7 * 7, 512), nn.ReLU())
        self.heads = nn.Linear(512, actions + 1)
        self.actions = actions

    def forward(self, observations):
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=observations.is_cuda):
            out = self.heads(self.trunk(observations.float() / 255.0)).float()
        return out[:, :self.actions], out[:, self.actions]


class RolloutLoop:
    """Collect ``horizon``-step rollouts from an environment and take one clipped
    policy-gradient pass over each."""

    def __init__(self, env, policy: NatureCnnPolicy, *, horizon: int = 16, gamma: float = 0.99, gae_lambda: float = 0.95,
                 learning_rate: float = 2.5e-4, clip: float = 0.1, minibatches: int = 4, seed: int = 0):
        self.env, self.policy = env, policy
        self.horizon, self.gamma, self.gae_lambda = horizon, gamma, gae_lambda
        self.clip, self.minibatches = clip, minibatches
        device, n = env.device, env.num_envs
        self.store = RolloutStore(horizon, n, device)
        self.reward = KillcountReward(n, device)
        self.optimizer = torch.optim.Adam(policy.parameters(), lr=learning_rate, eps=1e-5, capturable=True)
        torch.manual_seed(seed)              # the device's default generator drives sampling (it is graph-safe)
        self.lane_ids = torch.arange(n, device=device, dtype=torch.int64)
        self.reseeds = torch.zeros((), dtype=torch.int64, device=device)      # advanced on the device
        self.episode_starts = torch.ones(n, dtype=torch.bool, device=device)
        self.observations, _ = env.reset_device(torch.ones(n, dtype=torch.bool, device=device), self.lane_ids + 1 + seed)
        self.last_values = torch.zeros(n, device=device)
        self.last_dones = torch.zeros(n, dtype=torch.bool, device=device)

    @torch.no_grad()
    def act(self, observations):
        logits, values = self.policy(observations)
        # Gumbel-max sampling: a categorical draw without a host check of the probabilities
        noise = torch.rand_like(logits).clamp_min(1e-20)
        actions = torch.argmax(logits - torch.log(-torch.log(noise)), dim=1)
        log_probs = torch.log_softmax(logits, dim=1).gather(1, actions[:, None]).squeeze(1)
        return actions, values, log_probs

    def collect(self):
        """One rollout; returns the store (returns and advantages filled)."""

        env = self.env
        for step in range(self.horizon):
            actions, values, log_probs = self.act(self.observations)
            self.store.observations[step].copy_(self.observations)
            self.reseeds.add_(1)
            t = env.step_and_reset_device(actions, self.lane_ids + self.reseeds * env.num_envs)
            rewards = self.reward(t.final_signals, t.terminated, t.truncated)
            self.store.add(step, self.store.observations[step], self.episode_starts, actions, rewards, values, log_probs)
            self.episode_starts = t.terminated | t.truncated
            self.observations = t.observations
        _, last_values, _ = self.act(self.observations)
        self.last_values.copy_(last_values)
        self.last_dones.copy_(self.episode_starts)
        self.store.finish(self.last_values, self.last_dones, self.gamma, self.gae_lambda)
        return self.store

    def update(self):
        """One pass of clipped policy-gradient minibatches over the stored rollout; returns the
        mean loss (a device scalar)."""

        store = self.store
        total = store.n_steps * store.n_envs
        observations = store.observations.reshape(total, 4, 84, 84)
        actions, old_log_probs = store.actions.reshape(total), store.log_probs.reshape(total)
        advantages, returns = store.advantages.reshape(total), store.returns.reshape(total)
        order = torch.randperm(total, device=observations.device)
        losses = []
        for chunk in order.chunk(self.minibatches):
            logits, values = self.policy(observations[chunk])
            log_probs = torch.log_softmax(logits, dim=1).gather(1, actions[chunk, None]).squeeze(1)
            adv = advantages[chunk]
            adv = (adv - adv.mean()) / (adv.std() + 1e-8)
            ratio = torch.exp(log_probs - old_log_probs[chunk])
            policy_loss = -torch.minimum(ratio * adv, ratio.clamp(1 - self.clip, 1 + self.clip) * adv).mean()
            value_loss = 0.5 * (values - returns[chunk]).pow(2).mean()
            entropy = -(torch.softmax(logits, dim=1) * torch.log_softmax(logits, dim=1)).sum(dim=1).mean()
            loss = policy_loss + 0.5 * value_loss - 0.01 * entropy
            self.optimizer.zero_grad(set_to_none=False)
            loss.backward()
            nn.utils.clip_grad_norm_(self.policy.parameters(), 0.5)
            self.optimizer.step()
            losses.append(loss.detach())
        return torch.stack(losses).mean()
