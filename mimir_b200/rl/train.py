"""Training loops and evaluation (reference: rl/dqn.go: TrainDQN, rl/ppo.go: TrainPPO / Train, rl/rl.go:
Evaluate).  An environment has ``observations``, ``actions``, ``reset() -> obs`` and
``step(action) -> (obs, reward, done)``; a policy has ``greedy(obs) -> action``."""
from __future__ import annotations

from dataclasses import dataclass, field

from .agents import DQN, PPO


def evaluate(policy, env, episodes: int = 10, max_steps: int = 100_000) -> float:
    """The mean return of ``episodes`` episodes of ``policy`` acting greedily in ``env``."""
    total = 0.0
    for _ in range(episodes):
        obs, done, steps = env.reset(), False, 0
        while not done and steps < max_steps:
            obs, r, done = env.step(policy.greedy(obs))
            total += r
            steps += 1
    return total / max(episodes, 1)


@dataclass
class DQNConfig:
    steps: int = 5000               # environment steps in all
    hidden: int = 64
    lr: float = 1e-3
    gamma: float = 0.99
    buffer: int = 10000
    batch: int = 64
    target_every: int = 100
    eps: tuple = (1.0, 0.05, 2000)  # epsilon from, to, over how many steps
    double: bool = True
    seed: int = 0
    on_episode: object = None       # called with (episode, return) after each episode


def train_dqn(env, c: DQNConfig = DQNConfig()) -> DQN:
    """Epsilon-greedy Q-learning in ``env`` for ``c.steps`` steps."""
    if c.steps < 1 or c.batch < 1 or c.buffer < c.batch:
        raise ValueError("dqn: steps and batch must be positive and the buffer hold at least a batch")
    agent = DQN(env.observations, env.actions, hidden=c.hidden, lr=c.lr, gamma=c.gamma, buffer=c.buffer, batch=c.batch,
                target_every=c.target_every, eps=c.eps, double=c.double, seed=c.seed)
    obs, ret, episode = env.reset(), 0.0, 0
    for _ in range(c.steps):
        a = agent.act(obs)
        nxt, r, done = env.step(a)
        agent.observe(obs, a, r, nxt, done)
        obs, ret = nxt, ret + r
        if done:
            if c.on_episode is not None:
                c.on_episode(episode, ret)
            obs, ret, episode = env.reset(), 0.0, episode + 1
    return agent


@dataclass
class PPOConfig:
    updates: int = 30               # rollouts, each followed by ``epochs`` passes over it
    rollout: int = 256              # steps per environment per rollout
    envs: int = 4                   # environments stepped side by side
    hidden: int = 64
    lr: float = 3e-4
    gamma: float = 0.99
    lam: float = 0.95
    clip: float = 0.2
    epochs: int = 4
    minibatch: int = 64
    value_coef: float = 0.5
    entropy_coef: float = 0.01
    max_grad_norm: float = 0.5
    seed: int = 0
    on_update: object = None        # called with (update, stats)
    stats: list = field(default_factory=list)


def train(agent: PPO, envs: list, c: PPOConfig) -> PPO:
    """``c.updates`` rounds of: ``c.rollout`` steps in each environment (an episode that ends starts afresh),
    advantages per environment, then the clipped-surrogate update over all of them."""
    from .agents import gae
    import torch
    if not envs or c.updates < 1 or c.rollout < 1:
        raise ValueError("ppo: at least one environment, update and rollout step")
    obs = [e.reset() for e in envs]
    for u in range(c.updates):
        traj = [dict(obs=[], act=[], logp=[], rew=[], val=[], done=[]) for _ in envs]
        for _ in range(c.rollout):
            for k, e in enumerate(envs):
                a, lp, v = agent.act(obs[k])
                nxt, r, done = e.step(a)
                t = traj[k]
                t["obs"].append(obs[k]); t["act"].append(a); t["logp"].append(lp); t["rew"].append(r); t["val"].append(v); t["done"].append(done)
                obs[k] = e.reset() if done else nxt
        # one update over every environment's steps; each keeps its own bootstrap value
        all_obs, all_act, all_lp, all_adv, all_ret = [], [], [], [], []
        for k, t in enumerate(traj):
            last = 0.0 if t["done"][-1] else agent.act(obs[k])[2]
            adv, ret = gae(t["rew"], t["val"], t["done"], last, c.gamma, c.lam)
            all_obs += t["obs"]; all_act += t["act"]; all_lp += t["logp"]; all_adv += adv; all_ret += ret
        stats = agent.update_from(torch.tensor(all_obs, dtype=torch.float32), torch.tensor(all_act), torch.tensor(all_lp),
                                  torch.tensor(all_adv), torch.tensor(all_ret))
        c.stats.append(stats)
        if c.on_update is not None:
            c.on_update(u, stats)
    return agent


def train_ppo(new_env, c: PPOConfig = PPOConfig()) -> PPO:
    """``new_env(seed)`` makes each of the ``c.envs`` environments."""
    envs = [new_env(c.seed + k) for k in range(max(c.envs, 1))]
    agent = PPO(envs[0].observations, envs[0].actions, hidden=c.hidden, lr=c.lr, gamma=c.gamma, lam=c.lam, clip=c.clip, epochs=c.epochs,
                minibatch=c.minibatch, value_coef=c.value_coef, entropy_coef=c.entropy_coef, max_grad_norm=c.max_grad_norm, seed=c.seed)
    return train(agent, envs, c)
