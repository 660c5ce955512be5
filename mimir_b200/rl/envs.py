"""Environments with the classic dynamics (reference: rl/cartpole.go, rl/chain.go)."""
from __future__ import annotations

import math
import random


class CartPole:
    """Pole balancing (Barto, Sutton & Anderson): 4 observations, 2 actions, reward 1 per step,
    episode ends at |x| > 2.4, |theta| > 12 degrees or after ``max_steps``."""
    observations, actions = 4, 2

    def __init__(self, seed: int = 0, max_steps: int = 500):
        self.rng, self.max_steps = random.Random(seed), max_steps
        self.reset()

    def reset(self):
        self.state = [self.rng.uniform(-0.05, 0.05) for _ in range(4)]
        self.t = 0
        return list(self.state)

    def step(self, action: int):
        g, mc, mp, l, f, tau = 9.8, 1.0, 0.1, 0.5, 10.0, 0.02
        x, xd, th, thd = self.state
        force = f if action == 1 else -f
        ct, st = math.cos(th), math.sin(th)
        tmp = (force + mp * l * thd * thd * st) / (mc + mp)
        tha = (g * st - ct * tmp) / (l * (4.0 / 3.0 - mp * ct * ct / (mc + mp)))
        xa = tmp - mp * l * tha * ct / (mc + mp)
        x, xd, th, thd = x + tau * xd, xd + tau * xa, th + tau * thd, thd + tau * tha
        self.state, self.t = [x, xd, th, thd], self.t + 1
        done = abs(x) > 2.4 or abs(th) > 12 * math.pi / 180 or self.t >= self.max_steps
        return list(self.state), 1.0, done


class Chain:
    """N-state chain: action 1 moves right (reward 1 at the end), action 0 returns to the start
    with a small reward; tests exploration."""
    actions = 2

    def __init__(self, n: int = 5, small: float = 0.01, horizon: int = 50):
        self.n, self.small, self.horizon = n, small, horizon
        self.observations = n
        self.reset()

    def _obs(self):
        return [1.0 if i == self.s else 0.0 for i in range(self.n)]

    def reset(self):
        self.s, self.t = 0, 0
        return self._obs()

    def step(self, action: int):
        self.t += 1
        if action == 1:
            r = 1.0 if self.s == self.n - 1 else 0.0
            self.s = min(self.s + 1, self.n - 1)
        else:
            r, self.s = self.small, 0
        return self._obs(), r, self.t >= self.horizon
