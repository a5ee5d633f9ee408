"""Reinforcement learning: agents, buffers, environments, vectorised stepping, league."""
from .agents import (ActorCritic, ActorCriticConfig, ContinuousActorCritic, Dqn, DqnConfig, MultiAgentTrainer, Ppo,  # noqa: F401
                     PpoConfig, Sac, SacConfig)
from .core import (ButtonWorld, CartPole, Duel, Env, GridWorld, League, LineWorld, Mlp, MultiAgentEnv,  # noqa: F401
                   MultiAgentVectorEnv, PointMass, PrioritizedReplayBuffer, ReplayBuffer, RolloutBuffer, Space,
                   TeamButton, TurnLine, VectorEnv, gae)
