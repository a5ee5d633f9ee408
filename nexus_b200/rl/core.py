"""Reinforcement-learning building blocks: spaces, the `Mlp` with its own Adam, replay / prioritized /
rollout buffers, GAE, single-agent environments (native C++: LineWorld, GridWorld, CartPole, PointMass),
vectorised environments with persistent native worker threads, multi-agent environments (TeamButton,
ButtonWorld, Duel, TurnLine) and the ELO league.
Parity: include/nexus/rl/{space,mlp,replay_buffer,prioritized_replay,rollout_buffer,gae,envs,vector_env,
multi_agent,league}.hpp of the reference."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..nxs.archive import load_archive, save_archive


@dataclass(frozen=True)
class Space:
    kind: str            # "discrete" | "box"
    n: int               # actions (discrete) or dimensions (box)
    low: float = 0.0
    high: float = 1.0

    @staticmethod
    def discrete(n: int) -> "Space":
        return Space("discrete", n)

    @staticmethod
    def box(dim: int, low: float, high: float) -> "Space":
        return Space("box", dim, low, high)


class Mlp(torch.nn.Module):
    """Tanh MLP that carries its own Adam (step count + moments), as the agents store it in archives."""

    def __init__(self, sizes: Sequence[int], lr: float = 1e-3, seed: int = 0, out_gain: float = 1.0):
        super().__init__()
        self.sizes = [int(s) for s in sizes]
        g = torch.Generator().manual_seed(seed)
        self.layers = torch.nn.ModuleList()
        for i in range(len(sizes) - 1):
            lin = torch.nn.Linear(sizes[i], sizes[i + 1])
            bound = math.sqrt(6.0 / (sizes[i] + sizes[i + 1])) * (out_gain if i == len(sizes) - 2 else 1.0)
            with torch.no_grad():
                lin.weight.copy_((torch.rand(lin.weight.shape, generator=g) * 2 - 1) * bound)
                lin.bias.zero_()
            self.layers.append(lin)
        self.opt = torch.optim.Adam(self.parameters(), lr=lr)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for i, lin in enumerate(self.layers):
            x = lin(x)
            if i + 1 < len(self.layers):
                x = torch.tanh(x)
        return x

    def step(self, loss: torch.Tensor, clip: float = 0.0) -> None:
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        if clip > 0:
            torch.nn.utils.clip_grad_norm_(self.parameters(), clip)
        self.opt.step()

    # archive form ------------------------------------------------------------------------------
    def flat(self) -> np.ndarray:
        return torch.cat([p.detach().reshape(-1) for p in self.parameters()]).numpy().astype(np.float32)

    def load_flat(self, flat) -> None:
        flat = torch.as_tensor(np.asarray(flat, dtype=np.float32))
        off = 0
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(flat[off: off + p.numel()].view(p.shape))
                off += p.numel()

    def record(self, name: str) -> dict:
        m = []
        step = 0
        for p in self.parameters():
            st = self.opt.state.get(p, {})
            step = max(step, int(st.get("step", 0)))
            m.append(st.get("exp_avg", torch.zeros_like(p)).reshape(-1))
        for p in self.parameters():
            m.append(self.opt.state.get(p, {}).get("exp_avg_sq", torch.zeros_like(p)).reshape(-1))
        return {"name": name, "sizes": self.sizes, "adam_step": step, "parameters": self.flat(),
                "moments": torch.cat(m).detach().numpy().astype(np.float32)}

    def load_record(self, rec: dict) -> None:
        if [int(s) for s in rec["sizes"]] != self.sizes:
            raise ValueError(f"network {rec['name']}: sizes {list(rec['sizes'])} != {self.sizes}")
        self.load_flat(rec["parameters"])
        mom = torch.as_tensor(np.asarray(rec["moments"], dtype=np.float32))
        n = sum(p.numel() for p in self.parameters())
        if mom.numel() == 2 * n and int(rec["adam_step"]) > 0:
            off = 0
            for p in self.parameters():
                self.opt.state[p] = {"step": torch.tensor(float(rec["adam_step"])),
                                     "exp_avg": mom[off: off + p.numel()].view(p.shape).clone(),
                                     "exp_avg_sq": mom[n + off: n + off + p.numel()].view(p.shape).clone()}
                off += p.numel()


def save_agent(path: str, kind: str, config: Dict[str, object], nets: Dict[str, Mlp]) -> None:
    cfg = []
    for k, v in config.items():
        if isinstance(v, bool):
            cfg.append((k, 3, v))
        elif isinstance(v, int):
            cfg.append((k, 1, v))
        elif isinstance(v, float):
            cfg.append((k, 2, v))
        else:
            cfg.append((k, 4, str(v)))
    save_archive(path, {"layers": [], "weights": [], "optim": None, "trainer": None, "python": b"",
                        "rl": {"kind": kind, "config": cfg, "nets": [n.record(name) for name, n in nets.items()],
                               "elos": [], "player_weights": []}})


def load_agent_record(path: str, kind: str) -> Tuple[Dict[str, object], Dict[str, dict]]:
    a = load_archive(path)
    rl = a.get("rl")
    if rl is None or rl["kind"] != kind:
        raise ValueError(f"{path} holds no {kind!r} agent")
    return {k: v for k, _, v in rl["config"]}, {n["name"]: n for n in rl["nets"]}


# ------------------------------------------------------------------------------------------- buffers
class ReplayBuffer:
    def __init__(self, capacity: int, obs_dim: int, act_dim: int = 1, seed: int = 0):
        self.cap, self.n, self.pos = capacity, 0, 0
        self.obs = np.zeros((capacity, obs_dim), np.float32)
        self.next_obs = np.zeros((capacity, obs_dim), np.float32)
        self.act = np.zeros((capacity, act_dim), np.float32)
        self.rew = np.zeros(capacity, np.float32)
        self.done = np.zeros(capacity, np.float32)
        self.rng = np.random.default_rng(seed)

    def add(self, obs, act, rew, next_obs, done) -> int:
        i = self.pos
        self.obs[i], self.act[i], self.rew[i], self.next_obs[i], self.done[i] = obs, act, rew, next_obs, float(done)
        self.pos = (self.pos + 1) % self.cap
        self.n = min(self.n + 1, self.cap)
        return i

    def __len__(self):
        return self.n

    def _batch(self, idx):
        t = torch.from_numpy
        return {"obs": t(self.obs[idx]), "act": t(self.act[idx]), "rew": t(self.rew[idx]),
                "next_obs": t(self.next_obs[idx]), "done": t(self.done[idx]), "idx": idx}

    def sample(self, batch: int):
        return self._batch(self.rng.integers(0, self.n, size=batch))


class PrioritizedReplayBuffer(ReplayBuffer):
    """Proportional prioritisation with a sum tree (native: `csrc/host/rl_core.cpp`); stratified draws, one per segment
    of the total priority; importance weights ``(N p)^-beta / max``."""

    def __init__(self, capacity: int, obs_dim: int, act_dim: int = 1, alpha: float = 0.6, beta: float = 0.4,
                 eps: float = 1e-3, seed: int = 0):
        super().__init__(capacity, obs_dim, act_dim, seed)
        self.alpha, self.beta, self.eps = alpha, beta, eps
        self._tree = _native.SumTree(capacity)
        self.size = self._tree.leaves()
        self.max_p = 1.0

    def add(self, *a) -> int:
        i = super().add(*a)
        self._tree.set(i, self.max_p ** self.alpha)
        return i

    def sample(self, batch: int):
        total = self._tree.total()
        seg = total / batch
        lo = seg * np.arange(batch, dtype=np.float64)
        draws = self.rng.uniform(lo, lo + seg)
        idx, pr = self._tree.sample(draws, self.n)
        w = (self.n * (pr / total)) ** (-self.beta)
        out = self._batch(idx)
        out["weight"] = torch.from_numpy((w / w.max()).astype(np.float32))
        return out

    def update_priorities(self, idx, td_errors) -> None:
        e = np.abs(np.asarray(td_errors, dtype=np.float64)) + self.eps
        if e.size:
            self.max_p = max(self.max_p, float(e.max()))
        self._tree.set_many(np.asarray(idx, dtype=np.int64), e ** self.alpha)


def gae(rewards, values, dones, last_value: float, gamma: float = 0.99, lam: float = 0.95):
    """Generalised advantage estimation over one trajectory.  Returns (advantages, returns)."""
    return _native.gae(np.asarray(rewards, dtype=np.float64), np.asarray(values, dtype=np.float64),
                       np.asarray(dones, dtype=bool), float(last_value), gamma, lam)


class RolloutBuffer:
    def __init__(self):
        self.clear()

    def clear(self) -> None:
        self.obs, self.act, self.logp, self.rew, self.val, self.done = [], [], [], [], [], []

    def add(self, obs, act, logp, rew, val, done) -> None:
        self.obs.append(np.asarray(obs, np.float32))
        self.act.append(np.asarray(act, np.float32).reshape(-1))
        self.logp.append(float(logp))
        self.rew.append(float(rew))
        self.val.append(float(val))
        self.done.append(bool(done))

    def __len__(self):
        return len(self.rew)

    def finish(self, last_value: float, gamma: float, lam: float, normalize: bool = True):
        adv, ret = gae(self.rew, self.val, self.done, last_value, gamma, lam)
        if normalize and len(adv) > 1:
            adv = (adv - adv.mean()) / (adv.std() + 1e-8)
        t = torch.from_numpy
        return {"obs": t(np.stack(self.obs)), "act": t(np.stack(self.act)), "logp": torch.tensor(self.logp),
                "adv": t(adv.astype(np.float32)), "ret": t(ret.astype(np.float32)), "val": torch.tensor(self.val)}


# ------------------------------------------------------------------------------------------- environments
class Env:
    """Single native environment: LineWorld(length, horizon), GridWorld(size, horizon), CartPole, PointMass."""

    def __init__(self, kind: str, a: int = 0, b: int = 0):
        self._e = _native.NativeEnv(kind, a, b)
        self.kind = kind
        self.observation_space = Space.box(self._e.obs_dim, -math.inf, math.inf)
        self.action_space = Space.discrete(self._e.action_count) if self._e.discrete else \
            Space.box(self._e.action_count, -1.0, 1.0)

    def reset(self, seed: int = 0) -> np.ndarray:
        return self._e.reset(seed)

    def step(self, action):
        obs, r, term, trunc = self._e.step(np.atleast_1d(np.asarray(action, np.float32)))
        return obs, float(r), bool(term), bool(trunc)


def LineWorld(length: int = 5, horizon: int = 12) -> Env:
    return Env("LineWorld", length, horizon)


def GridWorld(size: int = 4, horizon: int = 24) -> Env:
    return Env("GridWorld", size, horizon)


def CartPole() -> Env:
    return Env("CartPole")


def PointMass() -> Env:
    return Env("PointMass")


class VectorEnv:
    """N copies stepped by persistent native worker threads; finished copies reset themselves."""

    def __init__(self, kind: str, count: int, a: int = 0, b: int = 0, workers: int = 0, seed: int = 0):
        self._v = _native.NativeVectorEnv(kind, count, a, b, workers, seed)
        self.size, self.obs_dim = self._v.size, self._v.obs_dim

    def reset(self):
        return self._v.reset()

    def step(self, actions):
        return self._v.step(np.asarray(actions, np.float32).reshape(self.size, -1))

    @property
    def total_steps(self) -> int:
        return self._v.total_steps


def _one_hot(i: int, n: int) -> np.ndarray:
    v = np.zeros(n, np.float32)
    v[i] = 1.0
    return v


class MultiAgentEnv:
    agents: List[str] = []
    simultaneous = True

    def observation_space(self, agent: str) -> Space:
        return self._obs_space

    def action_space(self, agent: str) -> Space:
        return Space.discrete(2)


class TeamButton(MultiAgentEnv):
    """Every agent has one button; the shared reward is 1 on steps where all are pressed."""

    def __init__(self, agent_count: int = 2, horizon: int = 6):
        if agent_count < 1:
            raise ValueError("TeamButton requires at least one agent")
        self.agents = [f"a{i}" for i in range(agent_count)]
        self.horizon, self._obs_space = horizon, Space.box(2, 0.0, 1.0)
        self.reset()

    def reset(self, seed: int = 0):
        self.pressed = [False] * len(self.agents)
        self.steps = 0
        return self._obs()

    def _obs(self):
        return {a: _one_hot(int(p), 2) for a, p in zip(self.agents, self.pressed)}

    def step(self, actions: Dict[str, int]):
        self.pressed = [int(actions[a]) == 1 for a in self.agents]
        self.steps += 1
        r = 1.0 if all(self.pressed) else 0.0
        stop = self.steps >= self.horizon
        return self._obs(), {a: r for a in self.agents}, {a: False for a in self.agents}, {a: stop for a in self.agents}, stop


class ButtonWorld(TeamButton):
    def __init__(self):
        super().__init__(2, 6)
        self.agents = ["a", "b"]
        self.reset()


class Duel(MultiAgentEnv):
    """One-step zero-sum matching game: ``a`` wins when the actions match."""

    def __init__(self):
        self.agents, self._obs_space = ["a", "b"], Space.box(1, 0.0, 1.0)

    def reset(self, seed: int = 0):
        return {a: np.ones(1, np.float32) for a in self.agents}

    def step(self, actions):
        s = 1.0 if int(actions["a"]) == int(actions["b"]) else -1.0
        return self.reset(), {"a": s, "b": -s}, {"a": True, "b": True}, {"a": False, "b": False}, True


class TurnLine(MultiAgentEnv):
    """Turn-based (agent-environment-cycle) walk on 0..4: action 0 moves right, 1 left; reward 1 at 4."""
    simultaneous = False

    def __init__(self):
        self.agents, self._obs_space = ["a", "b"], Space.box(1, 0.0, 4.0)
        self.reset()

    def reset(self, seed: int = 0):
        self.position, self.turn, self.last_reward = 0, 0, 0.0
        return self._obs()

    def _obs(self):
        return {a: np.array([float(self.position)], np.float32) for a in self.agents}

    def current_agent(self) -> str:
        return self.agents[self.turn]

    def step(self, actions):
        raise RuntimeError("TurnLine is turn-based; use step_one")

    def step_one(self, action: int) -> None:
        self.position = min(4, self.position + 1) if int(action) == 0 else max(0, self.position - 1)
        self.last_reward = 1.0 if self.position == 4 else 0.0
        self.turn = 1 - self.turn


class MultiAgentVectorEnv:
    def __init__(self, make, count: int):
        self.envs = [make() for _ in range(count)]
        self.agents = self.envs[0].agents

    def reset(self, seed: int = 0):
        return [e.reset(seed + i) for i, e in enumerate(self.envs)]

    def step(self, actions: List[Dict[str, int]]):
        out = []
        for e, a in zip(self.envs, actions):
            obs, rew, term, trunc, done = e.step(a)
            if done:
                obs = e.reset()
            out.append((obs, rew, term, trunc, done))
        return out


class League:
    """ELO-rated pool of frozen policies."""

    def __init__(self):
        self.players: List[dict] = []

    def add_player(self, elo: float = 1000.0) -> int:
        self.players.append({"elo": float(elo), "weights": None})
        return len(self.players) - 1

    def save(self, player: int, weights) -> None:
        self.players[player]["weights"] = np.asarray(weights, np.float32).copy()

    def weights(self, player: int) -> np.ndarray:
        w = self.players[player]["weights"]
        if w is None:
            raise LookupError("league player has no checkpoint")
        return w

    def result(self, first: int, second: int, score_first: float, k: float = 32.0) -> None:
        a, b = self.players[first], self.players[second]
        expected = 1.0 / (1.0 + 10.0 ** ((b["elo"] - a["elo"]) / 400.0))
        a["elo"] += k * (score_first - expected)
        b["elo"] += k * ((1.0 - score_first) - (1.0 - expected))

    def elo(self, player: int) -> float:
        return self.players[player]["elo"]

    def size(self) -> int:
        return len(self.players)

    def save_nxs(self, path: str) -> None:
        save_archive(path, {"layers": [], "weights": [], "optim": None, "trainer": None, "python": b"",
                            "rl": {"kind": "league", "config": [], "nets": [],
                                   "elos": [p["elo"] for p in self.players],
                                   "player_weights": [p["weights"] if p["weights"] is not None else np.zeros(0, np.float32)
                                                      for p in self.players]}})

    @staticmethod
    def load_nxs(path: str) -> "League":
        rl = load_archive(path).get("rl")
        if rl is None or rl["kind"] != "league":
            raise ValueError("nxs file is not a league")
        lg = League()
        for i, e in enumerate(rl["elos"]):
            pid = lg.add_player(e)
            if i < len(rl["player_weights"]) and len(rl["player_weights"][i]):
                lg.save(pid, rl["player_weights"][i])
        return lg
