"""Reinforcement learning (reference: rl/, examples/rl): CartPole and Chain environments, replay buffer,
DQN with a target network, PPO with GAE and the clipped surrogate, training loops over one or several
environments, and evaluation of a greedy policy."""
from .envs import CartPole, Chain  # noqa: F401
from .agents import DQN, PPO, ReplayBuffer, gae  # noqa: F401
from .train import DQNConfig, PPOConfig, evaluate, train, train_dqn, train_ppo  # noqa: F401
