"""The rollout loop around the environment (the benchmark definition's rollout workload):
reward, store, advantage estimate, and the render inside the loop."""

import numpy as np
import pytest
import torch

DEV = "cuda:0"


def test_generalised_advantage_estimate_known_answer(pkg):
    """Three steps, two lanes, gamma 0.5, lambda 0.5 worked by hand: a lane whose episode starts
    at step 2 does not bootstrap across the boundary; a finished last step ignores the last value."""

    from gradoom_b200 import rollout

    store = rollout.RolloutStore(3, 2, "cpu")
    store.rewards.copy_(torch.tensor([[1.0, 0.0], [0.0, 2.0], [1.0, 1.0]]))
    store.values.copy_(torch.tensor([[0.5, 1.0], [1.0, 0.0], [0.0, 2.0]]))
    store.episode_starts.copy_(torch.tensor([[True, True], [False, False], [False, True]]))
    store.finish(torch.tensor([4.0, 8.0]), torch.tensor([False, True]), 0.5, 0.5)
    # lane 0: delta2 = 1 + .5*4 - 0 = 3; delta1 = 0 + .5*0 - 1 = -1 -> A1 = -1 + .25*3 = -.25;
    #         delta0 = 1 + .5*1 - .5 = 1 -> A0 = 1 + .25*(-.25) = .9375
    # lane 1: done at the end: delta2 = 1 - 2 = -1; step 2 starts an episode: delta1 = 2 - 0 = 2, A1 = 2;
    #         delta0 = 0 + .5*0 - 1 = -1 -> A0 = -1 + .25*2 = -.5
    assert torch.allclose(store.advantages, torch.tensor([[0.9375, -0.5], [-0.25, 2.0], [3.0, -1.0]]))
    assert torch.allclose(store.returns, store.advantages + store.values)


def test_killcount_reward_counts_increments_per_episode(pkg):
    from gradoom_b200 import rollout

    reward = rollout.KillcountReward(3, "cpu")
    signals = torch.zeros((3, 27))
    no, yes = torch.zeros(3, dtype=torch.bool), torch.tensor([False, True, False])
    signals[:, 0] = torch.tensor([1.0, 2.0, 0.0])
    assert reward(signals, no, yes).tolist() == [1.0, 2.0, 0.0]           # lane 1's episode ends here
    signals[:, 0] = torch.tensor([3.0, 1.0, 0.0])
    assert reward(signals, no, no).tolist() == [2.0, 1.0, 0.0]            # lane 1 counts from zero again
    with pytest.raises(ValueError):
        rollout.KillcountReward(3, "cpu", signal_name="frags")


@pytest.mark.gpu
def test_identically_seeded_rollouts_agree_and_show_the_oracles_frames(pkg, oracle, scenes):
    from gradoom_b200 import rollout, scene as gdscene
    from gradoom_b200.env import GraDoomVecEnv

    sc, blob = scenes("c2")

    def run():
        env = GraDoomVecEnv(compiled_scenario=sc, num_envs=32, device=DEV, frame_skip=2, obs_crop=(0, 32, 0, 0),
                            obs_crop_mode="mask", max_things=12, producer_seed=5,
                            vizdoom_config={"episode_timeout": 40})
        torch.manual_seed(11)
        policy = rollout.NatureCnnPolicy().to(DEV)
        loop = rollout.RolloutLoop(env, policy, horizon=16, seed=11)
        first = loop.collect()
        returns, actions = first.returns.clone(), first.actions.clone()
        loss = loop.update()
        second = loop.collect()                      # crosses the 40-tic timeout: auto-resets inside the loop
        lanes, things = env._producer.render_inputs()
        newest = loop.observations[:, 3].cpu().numpy()
        expected = oracle.render(blob, lanes.cpu().numpy(), things.cpu().numpy())["obs"]
        env.check_status()
        env.close()
        return returns, actions, float(loss), second.returns.clone(), newest, expected, second.episode_starts.clone()

    a, b = run(), run()
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # the update's convolution gradients may be summed in another order: close, not equal
    assert np.isfinite(a[2]) and abs(a[2] - b[2]) < 1e-2 and bool(torch.isfinite(a[3]).all())
    assert np.array_equal(a[4], a[5])                # the loop's newest frames are the oracle's
    assert bool(a[6].any())                          # episodes did end and restart inside the rollout
    assert a[1].min() >= 0 and a[1].max() < 17 and len(torch.unique(a[1])) > 4
