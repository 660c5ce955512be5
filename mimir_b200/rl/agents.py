"""DQN and PPO on the nn / optim layers (reference: rl/dqn.go, rl/ppo.go)."""
from __future__ import annotations

import copy
import random

import torch

from .. import nn, optim
from .. import tensor as T


def mlp(sizes, act=nn.Tanh):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(act())
    return nn.Sequential(*layers)


class ReplayBuffer:
    def __init__(self, capacity: int, seed: int = 0):
        self.cap, self.data, self.pos, self.rng = capacity, [], 0, random.Random(seed)

    def add(self, *transition):
        if len(self.data) < self.cap:
            self.data.append(transition)
        else:
            self.data[self.pos] = transition
        self.pos = (self.pos + 1) % self.cap

    def sample(self, n: int):
        batch = self.rng.sample(self.data, n)
        return [torch.tensor(col, dtype=torch.float32) for col in zip(*batch)]

    def __len__(self):
        return len(self.data)


class DQN:
    """Q-learning with experience replay, a periodically copied target network, Huber loss and
    epsilon-greedy exploration (double-DQN target when ``double`` is set)."""

    def __init__(self, observations, actions, hidden=64, lr=1e-3, gamma=0.99, buffer=10000, batch=64, target_every=100,
                 eps=(1.0, 0.05, 2000), double=True, seed=0):
        nn.manual_seed(seed)
        self.q = mlp([observations, hidden, hidden, actions], nn.ReLU)
        self.target = copy.deepcopy(self.q)
        self.opt = optim.Adam(self.q.parameters(), lr=lr)
        self.buf, self.batch, self.gamma, self.actions = ReplayBuffer(buffer, seed), batch, gamma, actions
        self.target_every, self.eps, self.double, self.steps, self.rng = target_every, eps, double, 0, random.Random(seed)

    def epsilon(self):
        hi, lo, decay = self.eps
        return lo + (hi - lo) * max(0.0, 1 - self.steps / decay)

    def act(self, obs, greedy=False) -> int:
        if not greedy and self.rng.random() < self.epsilon():
            return self.rng.randrange(self.actions)
        return int(self.q(T.tensor([obs])).data().argmax())

    def greedy(self, obs) -> int:
        return self.act(obs, greedy=True)

    def values(self, obs) -> list:
        """The value of each action in ``obs``."""
        return self.q(T.tensor([obs])).data()[0].tolist()

    def observe(self, obs, action, reward, nxt, done):
        self.buf.add(obs, action, reward, nxt, float(done))
        self.steps += 1
        if len(self.buf) < self.batch:
            return None
        s, a, r, s2, d = self.buf.sample(self.batch)
        with torch.no_grad():
            q2 = self.target(T.from_torch(s2)).data()
            if self.double:
                best = self.q(T.from_torch(s2)).data().argmax(1, keepdim=True)
                nxt_v = q2.gather(1, best).squeeze(1)
            else:
                nxt_v = q2.max(1).values
            y = r + self.gamma * (1 - d) * nxt_v
        q = T.gather(self.q(T.from_torch(s)), 1, T.from_torch(a.long()[:, None]))
        loss = nn.loss.huber(T.reshape(q, (-1,)), T.from_torch(y))
        self.q.zero_grad()
        T.backward(loss)
        value = float(loss.data())   # read before the step overwrites the parameters the graph refers to
        self.opt.step()
        if self.steps % self.target_every == 0:
            self.target.load_state_dict({k: v.clone() for k, v in self.q.state_dict().items()})
        return value


def gae(rewards, values, dones, last_value, gamma=0.99, lam=0.95):
    """Generalised advantage estimates and returns for one rollout (lists of floats)."""
    adv, out, nxt = 0.0, [0.0] * len(rewards), last_value
    for t in reversed(range(len(rewards))):
        mask = 0.0 if dones[t] else 1.0
        delta = rewards[t] + gamma * nxt * mask - values[t]
        adv = delta + gamma * lam * mask * adv
        out[t], nxt = adv, values[t]
    return out, [a + v for a, v in zip(out, values)]


class PPO:
    """Clipped-surrogate PPO for discrete actions: shared rollout, several epochs of minibatches,
    value loss, entropy bonus, advantage normalisation, global-norm gradient clipping."""

    def __init__(self, observations, actions, hidden=64, lr=3e-4, gamma=0.99, lam=0.95, clip=0.2, epochs=4, minibatch=64,
                 value_coef=0.5, entropy_coef=0.01, max_grad_norm=0.5, seed=0):
        nn.manual_seed(seed)
        self.pi, self.v = mlp([observations, hidden, hidden, actions]), mlp([observations, hidden, hidden, 1])
        self.opt = optim.Adam(self.pi.parameters() + self.v.parameters(), lr=lr, clip_norm=max_grad_norm)
        self.gamma, self.lam, self.clip, self.epochs, self.mb = gamma, lam, clip, epochs, minibatch
        self.vc, self.ec, self.gen = value_coef, entropy_coef, torch.Generator().manual_seed(seed)

    def act(self, obs):
        with torch.no_grad():
            logits = self.pi(T.tensor([obs])).data()[0]
            value = float(self.v(T.tensor([obs])).data())
        probs = torch.softmax(logits, 0)
        a = int(torch.multinomial(probs, 1, generator=self.gen))
        return a, float(torch.log(probs[a])), value

    def probabilities(self, obs) -> list:
        """How likely the policy is to take each action in ``obs``."""
        return torch.softmax(self.pi(T.tensor([obs])).data()[0], 0).tolist()

    def greedy(self, obs) -> int:
        return int(self.pi(T.tensor([obs])).data()[0].argmax())

    def update(self, obs, actions, logps, rewards, values, dones, last_value):
        """One rollout of one environment: advantages by GAE, then ``update_from``."""
        adv, ret = gae(rewards, values, dones, last_value, self.gamma, self.lam)
        return self.update_from(torch.tensor(obs, dtype=torch.float32), torch.tensor(actions), torch.tensor(logps),
                                torch.tensor(adv), torch.tensor(ret))

    def update_from(self, obs, actions, old, adv, ret):
        """``epochs`` passes of minibatches over steps whose advantages and returns are given (tensors)."""
        adv = (adv - adv.mean()) / (adv.std() + 1e-8)
        stats = {}
        for _ in range(self.epochs):
            perm = torch.randperm(len(obs), generator=self.gen)
            for i in range(0, len(obs), self.mb):
                idx = perm[i:i + self.mb]
                logp_all = T.log_softmax(self.pi(T.from_torch(obs[idx])), -1)
                logp = T.reshape(T.gather(logp_all, 1, T.from_torch(actions[idx][:, None])), (-1,))
                ratio = T.exp(logp - T.from_torch(old[idx]))
                a = T.from_torch(adv[idx])
                surrogate = T.minimum(ratio * a, T.clamp(ratio, 1 - self.clip, 1 + self.clip) * a)
                entropy = -T.mean(T.sum_(T.exp(logp_all) * logp_all, -1))
                v = T.reshape(self.v(T.from_torch(obs[idx])), (-1,))
                vloss = T.mean((v - T.from_torch(ret[idx])) * (v - T.from_torch(ret[idx])))
                loss = -T.mean(surrogate) + self.vc * vloss - self.ec * entropy
                for m in (self.pi, self.v):
                    m.zero_grad()
                T.backward(loss)
                stats = {"loss": float(loss.data()), "value_loss": float(vloss.data()), "entropy": float(entropy.data())}
                self.opt.step()
        return stats
