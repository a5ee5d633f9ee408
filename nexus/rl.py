"""`nexus.rl`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.rl` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (Environment, LineWorld, GridWorld, CartPole, PointMass, VectorEnv, PPOConfig, PPOAgent, ActorCriticAgent, ContinuousActorCritic, ReplayBuffer, PrioritizedReplayBuffer, RolloutBuffer, League)  # noqa: F401

_native = _importlib.import_module("nexus_b200.rl")


def __getattr__(name):
    return getattr(_native, name)
