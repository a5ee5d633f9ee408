"""Self-play on the Duel game with an ELO league, and cooperative TeamButton with a shared policy (CPU)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200 import rl  # noqa: E402


def main():
    make = lambda: rl.ActorCritic(rl.ActorCriticConfig(obs_dim=2, actions=2, hidden=16, lr=3e-2))   # noqa: E731
    team = rl.MultiAgentTrainer(rl.TeamButton(3), make, shared=True)
    for ep in range(150):
        team.run_episode()
    print("TeamButton greedy return:", np.mean([team.run_episode(train=False, greedy=True)["a0"] for _ in range(5)]))
    make1 = lambda: rl.ActorCritic(rl.ActorCriticConfig(obs_dim=1, actions=2, hidden=8))   # noqa: E731
    league = rl.League()
    duel = rl.MultiAgentTrainer(rl.Duel(), make1, league=league, snapshot_every=20)
    for ep in range(200):
        duel.run_episode()
    print("league ratings:", [round(league.elo(i)) for i in range(league.size())])


if __name__ == "__main__":
    main()
