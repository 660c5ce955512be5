"""Training loops and evaluation (reference: rl/dqn.go, rl/ppo.go, rl/rl.go and their tests)."""
import pytest

from mimir_b200 import rl


def test_dqn_learns_to_walk_the_chain():
    env = rl.Chain(n=4, horizon=20)
    returns = []
    agent = rl.train_dqn(env, rl.DQNConfig(steps=2500, hidden=32, lr=5e-3, batch=32, target_every=50, eps=(1.0, 0.05, 600),
                                           on_episode=lambda i, r: returns.append(r)))
    assert rl.evaluate(agent, rl.Chain(n=4, horizon=20), episodes=3) >= 16         # walks right and collects at the end
    assert len(returns) == 125 and agent.greedy(env.reset()) == 1
    v = agent.values(env.reset())
    assert len(v) == 2 and v[1] > v[0]
    with pytest.raises(ValueError):
        rl.train_dqn(env, rl.DQNConfig(steps=0))


def test_ppo_balances_the_pole_over_several_environments():
    c = rl.PPOConfig(updates=25, rollout=128, envs=4, hidden=32, lr=3e-3, minibatch=128, seed=0)
    agent = rl.train_ppo(lambda seed: rl.CartPole(seed=seed, max_steps=200), c)
    score = rl.evaluate(agent, rl.CartPole(seed=99, max_steps=200), episodes=5)
    assert score > 100, score
    p = agent.probabilities([0.0, 0.0, 0.05, 0.5])                                  # the pole falls right: push right
    assert abs(sum(p) - 1) < 1e-5 and p[1] > 0.5 and len(c.stats) == 25 and "entropy" in c.stats[-1]
    with pytest.raises(ValueError):
        rl.train(agent, [], c)
