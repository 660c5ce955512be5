"""Reinforcement learning (reference: rl/, examples/rl): CartPole and Chain environments, replay
buffer, DQN with a target network, PPO with GAE and clipped surrogate."""
from .envs import CartPole, Chain
from .agents import DQN, PPO, ReplayBuffer, gae
