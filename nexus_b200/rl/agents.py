"""Agents: DQN (double / dueling / prioritized replay), PPO (clipped surrogate, value clipping, entropy
bonus, normalised GAE), SAC (twin critics, tanh-Gaussian policy, automatic temperature), ActorCritic
(one-step advantage) and ContinuousActorCritic (Gaussian policy); the multi-agent trainer (independent
learners, shared or separate policies, self-play against a league).
Parity: include/nexus/rl/{dqn,ppo,sac,actor_critic,multi_agent_trainer}.hpp of the reference."""
from __future__ import annotations

import copy
import math
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

from .core import (League, Mlp, PrioritizedReplayBuffer, ReplayBuffer, RolloutBuffer, load_agent_record, save_agent)


def _t(x) -> torch.Tensor:
    return torch.as_tensor(np.asarray(x, np.float32))


# ------------------------------------------------------------------------------------------------- DQN
@dataclass
class DqnConfig:
    obs_dim: int = 4
    actions: int = 2
    hidden: int = 64
    lr: float = 1e-3
    gamma: float = 0.99
    batch: int = 64
    buffer: int = 20000
    warmup: int = 200
    target_every: int = 200
    eps_start: float = 1.0
    eps_end: float = 0.05
    eps_steps: int = 3000
    double: bool = True
    dueling: bool = True
    prioritized: bool = False
    seed: int = 0


class Dqn:
    kind = "dqn"

    def __init__(self, cfg: DqnConfig):
        self.cfg = cfg
        out = cfg.actions + 1 if cfg.dueling else cfg.actions
        self.q = Mlp([cfg.obs_dim, cfg.hidden, cfg.hidden, out], cfg.lr, cfg.seed)
        self.target = copy.deepcopy(self.q)
        mk = PrioritizedReplayBuffer if cfg.prioritized else ReplayBuffer
        self.buf = mk(cfg.buffer, cfg.obs_dim, 1, seed=cfg.seed)
        self.rng = np.random.default_rng(cfg.seed)
        self.steps = 0

    def _qvalues(self, net: Mlp, obs: torch.Tensor) -> torch.Tensor:
        o = net(obs)
        if not self.cfg.dueling:
            return o
        v, a = o[..., :1], o[..., 1:]
        return v + a - a.mean(-1, keepdim=True)

    def epsilon(self) -> float:
        c = self.cfg
        return c.eps_end + (c.eps_start - c.eps_end) * max(0.0, 1.0 - self.steps / c.eps_steps)

    def act(self, obs, greedy: bool = False) -> int:
        if not greedy and self.rng.random() < self.epsilon():
            return int(self.rng.integers(self.cfg.actions))
        with torch.no_grad():
            return int(self._qvalues(self.q, _t(obs)[None]).argmax(-1))

    def observe(self, obs, act, rew, next_obs, done) -> Optional[float]:
        self.buf.add(obs, [act], rew, next_obs, done)
        self.steps += 1
        if len(self.buf) < max(self.cfg.warmup, self.cfg.batch):
            return None
        loss = self.update()
        if self.steps % self.cfg.target_every == 0:
            self.target.load_state_dict(self.q.state_dict())
        return loss

    def update(self) -> float:
        c = self.cfg
        b = self.buf.sample(c.batch)
        q = self._qvalues(self.q, b["obs"]).gather(1, b["act"].long())[:, 0]
        with torch.no_grad():
            nq_t = self._qvalues(self.target, b["next_obs"])
            if c.double:
                best = self._qvalues(self.q, b["next_obs"]).argmax(-1, keepdim=True)
                nq = nq_t.gather(1, best)[:, 0]
            else:
                nq = nq_t.max(-1).values
            target = b["rew"] + c.gamma * (1 - b["done"]) * nq
        td = q - target
        w = b.get("weight", torch.ones_like(td))
        loss = (w * F.smooth_l1_loss(q, target, reduction="none")).mean()
        self.q.step(loss, clip=10.0)
        if c.prioritized:
            self.buf.update_priorities(b["idx"], td.detach().numpy())
        return float(loss.detach())

    def save_nxs(self, path: str) -> None:
        save_agent(path, self.kind, asdict(self.cfg), {"q": self.q, "target": self.target})

    @staticmethod
    def load_nxs(path: str) -> "Dqn":
        cfg, nets = load_agent_record(path, "dqn")
        a = Dqn(DqnConfig(**cfg))
        a.q.load_record(nets["q"])
        a.target.load_record(nets["target"])
        return a


# ------------------------------------------------------------------------------------------------- PPO
@dataclass
class PpoConfig:
    obs_dim: int = 4
    actions: int = 2
    hidden: int = 64
    lr: float = 3e-3
    gamma: float = 0.99
    lam: float = 0.95
    clip: float = 0.2
    value_clip: float = 0.2
    value_coef: float = 0.5
    entropy_coef: float = 0.01
    epochs: int = 4
    minibatch: int = 64
    rollout: int = 256
    normalize_adv: bool = True
    seed: int = 0


class Ppo:
    kind = "ppo"

    def __init__(self, cfg: PpoConfig):
        self.cfg = cfg
        self.pi = Mlp([cfg.obs_dim, cfg.hidden, cfg.hidden, cfg.actions], cfg.lr, cfg.seed, out_gain=0.1)
        self.v = Mlp([cfg.obs_dim, cfg.hidden, cfg.hidden, 1], cfg.lr, cfg.seed + 1)
        self.buf = RolloutBuffer()
        self.gen = torch.Generator().manual_seed(cfg.seed)

    def act(self, obs, greedy: bool = False):
        with torch.no_grad():
            logits = self.pi(_t(obs)[None])[0]
            val = float(self.v(_t(obs)[None]))
            if greedy:
                a = int(logits.argmax())
            else:
                a = int(torch.multinomial(torch.softmax(logits, -1), 1, generator=self.gen))
            return a, float(torch.log_softmax(logits, -1)[a]), val

    def observe(self, obs, act, logp, rew, val, done, next_obs) -> Optional[dict]:
        self.buf.add(obs, [act], logp, rew, val, done)
        if len(self.buf) < self.cfg.rollout:
            return None
        with torch.no_grad():
            last = 0.0 if done else float(self.v(_t(next_obs)[None]))
        return self.update(last)

    def update(self, last_value: float) -> dict:
        c = self.cfg
        data = self.buf.finish(last_value, c.gamma, c.lam, c.normalize_adv)
        n = len(self.buf)
        self.buf.clear()
        stats = {}
        for _ in range(c.epochs):
            perm = torch.randperm(n, generator=self.gen)
            for s in range(0, n, c.minibatch):
                idx = perm[s: s + c.minibatch]
                logits = self.pi(data["obs"][idx])
                logp_all = torch.log_softmax(logits, -1)
                logp = logp_all.gather(1, data["act"][idx].long())[:, 0]
                ratio = torch.exp(logp - data["logp"][idx])
                adv = data["adv"][idx]
                surr = torch.min(ratio * adv, torch.clamp(ratio, 1 - c.clip, 1 + c.clip) * adv)
                entropy = -(logp_all.exp() * logp_all).sum(-1).mean()
                pi_loss = -surr.mean() - c.entropy_coef * entropy
                self.pi.step(pi_loss, clip=0.5)
                v = self.v(data["obs"][idx])[:, 0]
                v_clip = data["val"][idx] + torch.clamp(v - data["val"][idx], -c.value_clip, c.value_clip)
                v_loss = c.value_coef * torch.max((v - data["ret"][idx]) ** 2, (v_clip - data["ret"][idx]) ** 2).mean()
                self.v.step(v_loss, clip=0.5)
                stats = {"pi_loss": float(pi_loss), "v_loss": float(v_loss), "entropy": float(entropy),
                         "clip_frac": float(((ratio - 1).abs() > c.clip).float().mean())}
        return stats

    def save_nxs(self, path: str) -> None:
        save_agent(path, self.kind, asdict(self.cfg), {"pi": self.pi, "v": self.v})

    @staticmethod
    def load_nxs(path: str) -> "Ppo":
        cfg, nets = load_agent_record(path, "ppo")
        a = Ppo(PpoConfig(**cfg))
        a.pi.load_record(nets["pi"])
        a.v.load_record(nets["v"])
        return a


# ------------------------------------------------------------------------------------------------- SAC
@dataclass
class SacConfig:
    obs_dim: int = 2
    act_dim: int = 1
    hidden: int = 64
    lr: float = 3e-3
    gamma: float = 0.99
    tau: float = 0.01
    batch: int = 64
    buffer: int = 20000
    warmup: int = 200
    init_alpha: float = 0.2
    auto_alpha: bool = True
    seed: int = 0


class Sac:
    kind = "sac"

    def __init__(self, cfg: SacConfig):
        self.cfg = cfg
        io = cfg.obs_dim + cfg.act_dim
        self.pi = Mlp([cfg.obs_dim, cfg.hidden, cfg.hidden, 2 * cfg.act_dim], cfg.lr, cfg.seed, out_gain=0.1)
        self.q1 = Mlp([io, cfg.hidden, cfg.hidden, 1], cfg.lr, cfg.seed + 1)
        self.q2 = Mlp([io, cfg.hidden, cfg.hidden, 1], cfg.lr, cfg.seed + 2)
        self.t1, self.t2 = copy.deepcopy(self.q1), copy.deepcopy(self.q2)
        self.log_alpha = torch.tensor(math.log(cfg.init_alpha), requires_grad=True)
        self.alpha_opt = torch.optim.Adam([self.log_alpha], lr=cfg.lr)
        self.buf = ReplayBuffer(cfg.buffer, cfg.obs_dim, cfg.act_dim, seed=cfg.seed)
        self.gen = torch.Generator().manual_seed(cfg.seed)
        self.steps = 0

    def _sample(self, obs: torch.Tensor):
        mu, log_std = self.pi(obs).chunk(2, -1)
        log_std = log_std.clamp(-5, 2)
        eps = torch.randn(mu.shape, generator=self.gen)
        u = mu + log_std.exp() * eps
        a = torch.tanh(u)
        logp = (-0.5 * eps ** 2 - log_std - 0.5 * math.log(2 * math.pi)).sum(-1) - torch.log(1 - a ** 2 + 1e-6).sum(-1)
        return a, logp, torch.tanh(mu)

    def act(self, obs, greedy: bool = False) -> np.ndarray:
        with torch.no_grad():
            a, _, mean = self._sample(_t(obs)[None])
            return (mean if greedy else a)[0].numpy()

    def observe(self, obs, act, rew, next_obs, done) -> Optional[dict]:
        self.buf.add(obs, act, rew, next_obs, done)
        self.steps += 1
        if len(self.buf) < max(self.cfg.warmup, self.cfg.batch):
            return None
        return self.update()

    def update(self) -> dict:
        c = self.cfg
        b = self.buf.sample(c.batch)
        alpha = self.log_alpha.exp().detach()
        with torch.no_grad():
            na, nlogp, _ = self._sample(b["next_obs"])
            nx = torch.cat([b["next_obs"], na], -1)
            target = b["rew"] + c.gamma * (1 - b["done"]) * (torch.min(self.t1(nx), self.t2(nx))[:, 0] - alpha * nlogp)
        x = torch.cat([b["obs"], b["act"]], -1)
        l1, l2 = F.mse_loss(self.q1(x)[:, 0], target), F.mse_loss(self.q2(x)[:, 0], target)
        self.q1.step(l1)
        self.q2.step(l2)
        a, logp, _ = self._sample(b["obs"])
        xa = torch.cat([b["obs"], a], -1)
        pi_loss = (alpha * logp - torch.min(self.q1(xa), self.q2(xa))[:, 0]).mean()
        self.pi.step(pi_loss)
        if c.auto_alpha:
            al = -(self.log_alpha * (logp.detach() - c.act_dim).mean())
            self.alpha_opt.zero_grad()
            al.backward()
            self.alpha_opt.step()
        with torch.no_grad():
            for t, s in ((self.t1, self.q1), (self.t2, self.q2)):
                for pt, ps in zip(t.parameters(), s.parameters()):
                    pt.mul_(1 - c.tau).add_(ps, alpha=c.tau)
        return {"q_loss": float(l1 + l2), "pi_loss": float(pi_loss), "alpha": float(self.log_alpha.exp())}

    def save_nxs(self, path: str) -> None:
        cfg = asdict(self.cfg)
        cfg["init_alpha"] = float(self.log_alpha.exp())
        save_agent(path, self.kind, cfg, {"pi": self.pi, "q1": self.q1, "q2": self.q2, "t1": self.t1, "t2": self.t2})

    @staticmethod
    def load_nxs(path: str) -> "Sac":
        cfg, nets = load_agent_record(path, "sac")
        a = Sac(SacConfig(**cfg))
        for name in ("pi", "q1", "q2", "t1", "t2"):
            getattr(a, name).load_record(nets[name])
        return a


# ------------------------------------------------------------------------------------------------- actor-critic
@dataclass
class ActorCriticConfig:
    obs_dim: int = 4
    actions: int = 2       # discrete: number of actions; continuous: action dimensions
    hidden: int = 64
    lr: float = 3e-3
    gamma: float = 0.99
    entropy_coef: float = 0.01
    seed: int = 0


class ActorCritic:
    """One-step advantage actor-critic with a categorical policy."""
    kind = "actor_critic"

    def __init__(self, cfg: ActorCriticConfig):
        self.cfg = cfg
        self.pi = Mlp([cfg.obs_dim, cfg.hidden, cfg.actions], cfg.lr, cfg.seed, out_gain=0.1)
        self.v = Mlp([cfg.obs_dim, cfg.hidden, 1], cfg.lr, cfg.seed + 1)
        self.gen = torch.Generator().manual_seed(cfg.seed)

    def act(self, obs, greedy: bool = False) -> int:
        with torch.no_grad():
            logits = self.pi(_t(obs)[None])[0]
            return int(logits.argmax()) if greedy else int(torch.multinomial(torch.softmax(logits, -1), 1, generator=self.gen))

    def observe(self, obs, act, rew, next_obs, done) -> float:
        c = self.cfg
        o, no = _t(obs)[None], _t(next_obs)[None]
        with torch.no_grad():
            target = rew + (0.0 if done else c.gamma * float(self.v(no)))
        v = self.v(o)[0, 0]
        adv = target - float(v.detach())
        self.v.step((v - target) ** 2)
        lp = torch.log_softmax(self.pi(o)[0], -1)
        ent = -(lp.exp() * lp).sum()
        self.pi.step(-(lp[int(act)] * adv) - c.entropy_coef * ent)
        return adv

    def save_nxs(self, path: str) -> None:
        save_agent(path, self.kind, asdict(self.cfg), {"pi": self.pi, "v": self.v})

    @classmethod
    def load_nxs(cls, path: str):
        cfg, nets = load_agent_record(path, cls.kind)
        a = cls(ActorCriticConfig(**cfg))
        a.pi.load_record(nets["pi"])
        a.v.load_record(nets["v"])
        return a


class ContinuousActorCritic(ActorCritic):
    """Gaussian policy (state-independent log std) for box action spaces."""
    kind = "continuous_actor_critic"

    def __init__(self, cfg: ActorCriticConfig):
        super().__init__(cfg)
        self.log_std = torch.zeros(cfg.actions, requires_grad=True)
        self.std_opt = torch.optim.Adam([self.log_std], lr=cfg.lr)

    def act(self, obs, greedy: bool = False) -> np.ndarray:
        with torch.no_grad():
            mu = self.pi(_t(obs)[None])[0]
            if greedy:
                return mu.numpy()
            return (mu + self.log_std.exp() * torch.randn(mu.shape, generator=self.gen)).numpy()

    def observe(self, obs, act, rew, next_obs, done) -> float:
        c = self.cfg
        o, no = _t(obs)[None], _t(next_obs)[None]
        with torch.no_grad():
            target = rew + (0.0 if done else c.gamma * float(self.v(no)))
        v = self.v(o)[0, 0]
        adv = target - float(v.detach())
        self.v.step((v - target) ** 2)
        mu = self.pi(o)[0]
        a = _t(act)
        logp = (-0.5 * ((a - mu) / self.log_std.exp()) ** 2 - self.log_std - 0.5 * math.log(2 * math.pi)).sum()
        self.std_opt.zero_grad()
        self.pi.step(-logp * adv)
        self.std_opt.step()
        with torch.no_grad():
            self.log_std.clamp_(-3, 1)
        return adv


# ------------------------------------------------------------------------------------------------- multi-agent
class MultiAgentTrainer:
    """Independent learners on a multi-agent environment.  ``shared=True`` trains one policy for all
    agents; with a ``league`` the opponent of a two-player zero-sum game is sampled from frozen snapshots
    and ratings are updated after every episode."""

    def __init__(self, env, make_agent, shared: bool = False, league: Optional[League] = None, snapshot_every: int = 50):
        self.env, self.shared, self.league, self.snapshot_every = env, shared, league, snapshot_every
        proto = make_agent()
        self.agents: Dict[str, object] = {a: (proto if shared else (proto if i == 0 else make_agent()))
                                          for i, a in enumerate(env.agents)}
        self.episodes = 0
        self.learner_id = league.add_player() if league is not None else None
        self._make = make_agent

    def run_episode(self, train: bool = True, greedy: bool = False) -> Dict[str, float]:
        env = self.env
        obs = env.reset(self.episodes)
        totals = {a: 0.0 for a in env.agents}
        opponent, opp_id = None, None
        if self.league is not None and self.league.size() > 1 and len(env.agents) == 2:
            cands = [i for i in range(self.league.size()) if i != self.learner_id and self.league.players[i]["weights"] is not None]
            if cands:
                opp_id = cands[self.episodes % len(cands)]
                opponent = self._make()
                opponent.pi.load_flat(self.league.weights(opp_id))
        done = False
        while not done:
            if env.simultaneous:
                acts, extra = {}, {}
                for i, a in enumerate(env.agents):
                    ag = opponent if (opponent is not None and i == 1) else self.agents[a]
                    out = ag.act(obs[a], greedy=greedy)
                    acts[a], extra[a] = (out[0], out[1:]) if isinstance(out, tuple) else (out, ())
                nobs, rew, term, trunc, done = env.step(acts)
                for i, a in enumerate(env.agents):
                    totals[a] += rew[a]
                    if train and not (opponent is not None and i == 1):
                        d = term[a] or trunc[a]
                        ag = self.agents[a]
                        if extra[a]:
                            ag.observe(obs[a], acts[a], extra[a][0], rew[a], extra[a][1], d, nobs[a])
                        else:
                            ag.observe(obs[a], acts[a], rew[a], nobs[a], d)
                obs = nobs
            else:
                a = env.current_agent()
                out = self.agents[a].act(obs[a], greedy=greedy)
                act = out[0] if isinstance(out, tuple) else out
                env.step_one(act)
                nobs = env._obs()
                r = env.last_reward
                totals[a] += r
                done = r > 0 or sum(abs(v) for v in totals.values()) > 50 or getattr(env, "_n", 0) > 40
                env._n = getattr(env, "_n", 0) + 1
                if train:
                    ag = self.agents[a]
                    if isinstance(out, tuple):
                        ag.observe(obs[a], act, out[1], r, out[2], done, nobs[a])
                    else:
                        ag.observe(obs[a], act, r, nobs[a], done)
                obs = nobs
                if done:
                    env._n = 0
        self.episodes += 1
        if self.league is not None:
            first = env.agents[0]
            if opp_id is not None:
                score = 1.0 if totals[first] > 0 else (0.5 if totals[first] == 0 else 0.0)
                self.league.result(self.learner_id, opp_id, score)
            if self.episodes % self.snapshot_every == 0:
                pid = self.league.add_player(self.league.elo(self.learner_id))
                self.league.save(pid, self.agents[first].pi.flat())
        return totals
