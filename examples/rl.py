"""PPO on CartPole and DQN on the chain environment (reference: examples/rl/ppo, examples/rl/dqn)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def ppo_main(iterations=15, horizon=512, log=print):
    from mimir_b200 import rl
    env, agent = rl.CartPole(seed=0, max_steps=200), rl.PPO(4, 2, hidden=32, lr=3e-3, minibatch=128)
    lengths = []
    for it in range(iterations):
        O, A, L, R, V, D = [], [], [], [], [], []
        obs, ep = env.reset(), 0
        for _ in range(horizon):
            a, lp, v = agent.act(obs)
            nxt, r, done = env.step(a)
            O.append(obs); A.append(a); L.append(lp); R.append(r); V.append(v); D.append(done)
            obs, ep = nxt, ep + 1
            if done:
                lengths.append(ep)
                obs, ep = env.reset(), 0
        agent.update(O, A, L, R, V, D, agent.act(obs)[2])
        log(f"ppo iteration {it + 1}: mean episode length {sum(lengths[-10:]) / max(1, len(lengths[-10:])):.1f}")
    return lengths


def dqn_main(episodes=60, log=print):
    from mimir_b200 import rl
    env = rl.Chain(n=4, horizon=20)
    agent = rl.DQN(env.observations, env.actions, hidden=32, lr=5e-3, batch=32, target_every=50, eps=(1.0, 0.05, 600))
    returns = []
    for _ in range(episodes):
        obs, done, total = env.reset(), False, 0.0
        while not done:
            a = agent.act(obs)
            nxt, r, done = env.step(a)
            agent.observe(obs, a, r, nxt, done)
            obs, total = nxt, total + r
        returns.append(total)
    log(f"dqn: mean return of the last 10 episodes {sum(returns[-10:]) / 10:.1f}")
    return returns


if __name__ == "__main__":
    ppo_main()
    dqn_main()
