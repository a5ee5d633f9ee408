import numpy as np
import pytest
import torch

from nexus_b200 import rl


def run_single(agent, env, episodes, ppo=False):
    returns = []
    for ep in range(episodes):
        obs, done, total = env.reset(ep), False, 0.0
        while not done:
            if ppo:
                a, logp, val = agent.act(obs)
                nobs, r, term, trunc = env.step(a)
                agent.observe(obs, a, logp, r, val, term or trunc, nobs)
            else:
                a = agent.act(obs)
                nobs, r, term, trunc = env.step(a)
                agent.observe(obs, a, r, nobs, term)
            obs, total, done = nobs, total + r, term or trunc
        returns.append(total)
    return returns


def greedy_return(agent, env, limit=50):
    """Return of the greedy policy (LineWorld pays 0.1 per step to the right and 1 at the goal, so the
    straight path is worth 1.4 and a policy that never reaches the goal at most 0.3)."""
    obs, n, total = env.reset(0), 0, 0.0
    while n < limit:
        out = agent.act(obs, greedy=True)
        obs, r, term, trunc = env.step(out[0] if isinstance(out, tuple) else out)
        n, total = n + 1, total + r
        if term or trunc:
            break
    return total


def test_gae_and_buffers():
    adv, ret = rl.gae([1, 1, 1], [0.5, 0.5, 0.5], [False, False, True], 9.0, gamma=0.9, lam=1.0)
    assert np.allclose(ret, [1 + 0.9 + 0.81, 1.9, 1.0], atol=1e-6) and np.allclose(adv, ret - 0.5, atol=1e-6)
    b = rl.ReplayBuffer(4, 2)
    for i in range(6):
        b.add([i, i], [i % 2], float(i), [i + 1, i + 1], i == 5)
    assert len(b) == 4 and set(b.sample(32)["rew"].tolist()) <= {2.0, 3.0, 4.0, 5.0}
    p = rl.PrioritizedReplayBuffer(8, 1, alpha=1.0, beta=1.0, seed=1)
    for i in range(8):
        p.add([i], [0], 0.0, [i], False)
    p.update_priorities(np.arange(8), np.array([0, 0, 0, 0, 0, 0, 0, 100.0]))
    s = p.sample(64)
    assert (s["idx"] == 7).mean() > 0.8 and float(s["weight"].max()) == 1.0
    r = rl.RolloutBuffer()
    for t in range(5):
        r.add([t], [0], -0.7, 1.0, 0.0, t == 4)
    d = r.finish(0.0, 0.99, 0.95)
    assert d["obs"].shape == (5, 1) and abs(float(d["adv"].mean())) < 1e-6


def test_dqn_learns_lineworld_and_round_trips(tmp_path):
    env = rl.LineWorld(5, 12)
    agent = rl.Dqn(rl.DqnConfig(obs_dim=5, actions=2, hidden=32, eps_steps=600, warmup=64, batch=32, target_every=50,
                                lr=3e-3, prioritized=True, gamma=0.9, seed=0))
    run_single(agent, env, 120)
    assert greedy_return(agent, env) >= 1.39
    p = str(tmp_path / "dqn.nxs")
    agent.save_nxs(p)
    again = rl.Dqn.load_nxs(p)
    obs = env.reset(0)
    assert again.act(obs, greedy=True) == agent.act(obs, greedy=True)
    assert torch.equal(again.q.layers[0].weight, agent.q.layers[0].weight) and again.cfg.prioritized
    with pytest.raises(ValueError):
        rl.Ppo.load_nxs(p)


def test_ppo_improves_on_cartpole(tmp_path):
    env = rl.CartPole()
    agent = rl.Ppo(rl.PpoConfig(obs_dim=4, actions=2, hidden=32, rollout=256, minibatch=64, epochs=4, lr=3e-3, seed=1))
    ret = run_single(agent, env, 120, ppo=True)
    assert np.mean(ret[-20:]) > 1.5 * np.mean(ret[:20])
    p = str(tmp_path / "ppo.nxs")
    agent.save_nxs(p)
    again = rl.Ppo.load_nxs(p)
    assert torch.equal(again.pi.layers[-1].weight, agent.pi.layers[-1].weight)
    assert again.pi.opt.state[again.pi.layers[0].weight]["step"] > 0


def test_sac_and_continuous_actor_critic_on_pointmass(tmp_path):
    env = rl.PointMass()
    sac = rl.Sac(rl.SacConfig(obs_dim=env.observation_space.n, act_dim=1, hidden=32, warmup=64, batch=32, seed=0))
    ret = run_single(sac, env, 30)
    assert np.isfinite(ret).all() and np.mean(ret[-5:]) >= np.mean(ret[:5]) - 1e-3
    p = str(tmp_path / "sac.nxs")
    sac.save_nxs(p)
    assert np.allclose(rl.Sac.load_nxs(p).act(env.reset(0), greedy=True), sac.act(env.reset(0), greedy=True), atol=1e-6)
    cac = rl.ContinuousActorCritic(rl.ActorCriticConfig(obs_dim=env.observation_space.n, actions=1, hidden=16))
    assert np.isfinite(run_single(cac, env, 5)).all()
    ac = rl.ActorCritic(rl.ActorCriticConfig(obs_dim=5, actions=2, hidden=16, lr=1e-2, gamma=0.9))
    run_single(ac, rl.LineWorld(5, 12), 150)
    assert greedy_return(ac, rl.LineWorld(5, 12)) >= 1.39


def test_vector_env_and_multi_agent_envs():
    v = rl.VectorEnv("LineWorld", 6, 5, 12, workers=2, seed=3)
    obs = v.reset()
    assert obs.shape == (6, 5)
    for _ in range(30):
        out = v.step(np.zeros((6, 1), np.float32))
    assert v.total_steps == 180
    tb = rl.TeamButton(3)
    tb.reset()
    obs, rew, term, trunc, done = tb.step({"a0": 1, "a1": 1, "a2": 0})
    assert rew["a0"] == 0.0 and obs["a2"].tolist() == [1.0, 0.0]
    obs, rew, *_ = tb.step({"a0": 1, "a1": 1, "a2": 1})
    assert rew["a1"] == 1.0
    d = rl.Duel()
    _, rew, term, _, done = d.step({"a": 1, "b": 1})
    assert rew == {"a": 1.0, "b": -1.0} and done
    t = rl.TurnLine()
    with pytest.raises(RuntimeError):
        t.step({})
    for _ in range(4):
        t.step_one(0)
    assert t.position == 4 and t.last_reward == 1.0 and t.current_agent() == "a"
    mv = rl.MultiAgentVectorEnv(rl.ButtonWorld, 3)
    mv.reset()
    assert len(mv.step([{"a": 1, "b": 1}] * 3)) == 3


def test_league_elo_and_multi_agent_trainer(tmp_path):
    lg = rl.League()
    a, b = lg.add_player(), lg.add_player(1200.0)
    lg.result(a, b, 1.0)
    assert lg.elo(a) > 1000 and lg.elo(b) < 1200 and abs((lg.elo(a) - 1000) + (lg.elo(b) - 1200)) < 1e-4
    lg.save(a, [1.0, 2.0])
    p = str(tmp_path / "l.nxs")
    lg.save_nxs(p)
    l2 = rl.League.load_nxs(p)
    assert l2.size() == 2 and np.allclose(l2.weights(0), [1, 2]) and abs(l2.elo(1) - lg.elo(b)) < 1e-3
    with pytest.raises(LookupError):
        l2.weights(1)
    make = lambda: rl.ActorCritic(rl.ActorCriticConfig(obs_dim=2, actions=2, hidden=8, lr=3e-2))   # noqa: E731
    tr = rl.MultiAgentTrainer(rl.ButtonWorld(), make, shared=True)
    first = np.mean([tr.run_episode()["a"] for _ in range(10)])
    for _ in range(80):
        tr.run_episode()
    last = np.mean([tr.run_episode(train=False, greedy=True)["a"] for _ in range(5)])
    assert last >= first and last >= 4.0
    make1 = lambda: rl.ActorCritic(rl.ActorCriticConfig(obs_dim=1, actions=2, hidden=8))   # noqa: E731
    duel = rl.MultiAgentTrainer(rl.Duel(), make1, league=rl.League(), snapshot_every=5)
    for _ in range(20):
        duel.run_episode()
    assert duel.league.size() >= 4


def test_native_sum_tree_and_gae():
    from nexus_b200 import _native
    t = _native.SumTree(5)
    assert t.leaves() == 8 and t.total() == 0.0
    for i, p in enumerate([1.0, 0.0, 2.0, 0.5, 4.0]):
        t.set(i, p)
    assert t.total() == 7.5 and [t.find(x) for x in (0.5, 1.0, 1.5, 3.0, 3.2, 3.6, 7.5)] == [0, 0, 2, 2, 3, 4, 4]
    t.set_many(np.array([0, 4]), np.array([0.0, 1.0]))
    assert t.total() == 3.5 and t.find(0.1) == 2 and t.get(4) == 1.0
    idx, pr = t.sample(np.array([0.1, 2.2, 3.4]), 5)
    assert idx.tolist() == [2, 3, 4] and pr.tolist() == [2.0, 0.5, 1.0]
    assert t.sample(np.array([3.4]), 3)[0].tolist() == [2]               # capped at the last written slot
    with pytest.raises(IndexError):
        t.set(8, 1.0)
    with pytest.raises(ValueError):
        t.set(0, -1.0)
    # stratified sampling follows the priorities
    big = _native.SumTree(1000)
    pri = np.random.default_rng(0).random(1000) ** 3
    big.set_many(np.arange(1000), pri)
    draws = np.random.default_rng(1).uniform(0, big.total(), 200000)
    counts = np.bincount(big.sample(draws, 1000)[0], minlength=1000)
    assert np.abs(counts / counts.sum() - pri / pri.sum()).max() < 2e-3
    # gae: closed form on a constant-reward episode and the episode boundary
    adv, ret = _native.gae(np.ones(4), np.zeros(4), np.array([False, True, False, False]), 2.0, 0.5, 1.0)
    assert np.allclose(ret, [1.5, 1.0, 1 + 0.5 * (1 + 0.5 * 2.0), 1 + 0.5 * 2.0]) and np.allclose(adv, ret)
    with pytest.raises(ValueError):
        _native.gae(np.ones(3), np.zeros(4), np.zeros(3, dtype=bool), 0.0)
