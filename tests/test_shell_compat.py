"""Scripts written against the reference's Python shell (`import nexus`) run unchanged: every call below uses only the
`nexus` package with the reference's signatures (flat lists, `nexus.Tensor`, explicit forward / backward, parameter
records, builders).  The scenarios are those of the reference's python/tests (test_kabuk.py, test_faz1/2/4/5/6/7.py,
test_graph_lm.py): classifier + archive round trip, python-defined activations and modules that survive a fresh
process, images, GEMM, agents, buffers, tapes, graphs and the small language trainer."""
import math
import os
import subprocess
import sys

import pytest

import nexus

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _fresh_process(code: str) -> subprocess.CompletedProcess:
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)


# ------------------------------------------------------------------------------------------- trainer + archive
def test_classifier_trains_and_round_trips_through_an_archive(tmp_path):
    feats, labels = [], []
    for i in range(32):
        x = 1.0 if i % 2 == 0 else -1.0
        feats += [x, 0.0]
        labels.append(1 if x > 0 else 0)
    model = nexus.nn.Sequential()
    model.add(nexus.nn.Linear(2, 8, True))
    model.add(nexus.nn.swish())
    model.add(nexus.nn.Linear(8, 2, True))
    trainer = (nexus.train.TrainerBuilder(model).adamw(model, lr=0.08).loss(0.0).execution_policy_cpu()
               .gradient_clip_norm(1.0).accuracy().build())
    loader = nexus.data.DataLoader(feats, labels, 2, 8, False, 1)
    trainer.fit(loader, loader, 8)
    hist = trainer.history()
    assert hist[-1].train_loss < hist[0].train_loss
    path = str(tmp_path / "net.nxs")
    model.save_nxs(path)
    again = nexus.load(path)
    x = nexus.Tensor([1, 2])
    x[0], x[1] = 1.0, 0.0
    a, b = model.forward(x).to_list(), again.forward(x).to_list()
    assert max(abs(p - q) for p, q in zip(a, b)) < 1e-5


def test_parameters_alias_the_model_storage():
    model = nexus.nn.Sequential()
    model.add(nexus.nn.Linear(2, 3, True))
    params = model.parameters()
    assert len(params) == 2
    values = params[0]["values"]
    n = len(values.to_list())
    values.copy_from([1.0] * n)
    assert model.parameters()[0]["values"].to_list() == [1.0] * n
    model.zero_grad()


def test_optimizer_loss_and_metric_on_flat_lists():
    model = nexus.nn.Sequential()
    model.add(nexus.nn.Linear(2, 2, True))
    opt = nexus.optim.SGD(model, lr=0.1, momentum=0.0, weight_decay=0.0)
    assert abs(opt.learning_rate() - 0.1) < 1e-6
    opt.set_learning_rate(0.02)
    assert abs(opt.learning_rate() - 0.02) < 1e-6
    opt.zero_grad()
    out = nexus.loss.CrossEntropy(0.0).forward_backward([2.0, 0.0, 0.0, 2.0], [0, 1], 2)
    assert out["loss"] > 0.0 and len(out["grad"]) == 4
    acc = nexus.metrics.Accuracy()
    acc.update([2.0, 0.0, 0.0, 2.0], [0, 1], 2)
    assert abs(acc.value() - 1.0) < 1e-6
    acc.reset()
    assert acc.value() == 0.0
    loss, grad = nexus.loss.MSE().forward_backward([1.0, 2.0], [1.0, 0.0])
    assert loss > 0.0 and len(grad) == 2


def test_loader_schedule_logger_and_callbacks():
    loader = nexus.data.DataLoader([1.0, 0.0, 0.0, 1.0], [0, 1], 2, 1, False, 1)
    assert loader.features_per_sample() == 2
    assert loader.next()["batch_size"] == 1
    assert loader.next()["labels"] == [1]
    assert loader.next() is None
    loader.reset()
    assert loader.next()["labels"] == [0]
    model = nexus.nn.Sequential()
    model.add(nexus.nn.Linear(2, 2, True))
    logger = nexus.train.ProgressLogger()
    trainer = (nexus.train.TrainerBuilder(model).adamw(model, lr=0.1).loss().cosine(nexus.optim.CosineAnnealing(0.1, 2))
               .callback(logger).mixed_precision(False).build())
    trainer.fit(loader, loader, 1)
    assert logger.last()["epoch"] == 0

    class StopAfterOne(nexus.train.Callback):
        def __init__(self):
            super().__init__()
            self.epochs = []

        def on_epoch_end(self, state):
            self.epochs.append(state["epoch"])

        def stop(self):
            return len(self.epochs) >= 1

    watch = StopAfterOne()
    model2 = nexus.nn.Sequential()
    model2.add(nexus.nn.Linear(2, 2, True))
    t2 = nexus.train.TrainerBuilder(model2).adamw(model2, lr=0.05).loss().callback(watch).build()
    t2.fit(loader, loader, 4)
    assert watch.epochs == [0] and t2.epochs_ran() == 1


# ------------------------------------------------------------------------ python bodies inside archives
def test_named_activation_survives_a_fresh_process_and_rejects_object_closures(tmp_path):
    def double(x):
        return x * 2

    model = nexus.nn.Sequential()
    model.add(nexus.nn.activation("Double", double))
    x = nexus.Tensor([2])
    x.copy_from([1.5, -0.5])
    first = model.forward(x).to_list()
    path = str(tmp_path / "act.nxs")
    model.save_nxs(path)
    assert max(abs(a - b) for a, b in zip(first, nexus.load(path).forward(x).to_list())) < 1e-5
    r = _fresh_process(f"import nexus\nm = nexus.load({path!r})\nx = nexus.Tensor([2])\nx.copy_from([1.5, -0.5])\n"
                       "print(m.forward(x).to_list())\n")
    assert r.returncode == 0, r.stderr
    assert "3.0" in r.stdout and "-1.0" in r.stdout

    def closes_over_a_list():
        box = [3.0]
        return lambda x: x * box[0]

    with pytest.raises(TypeError, match="kapali"):
        nexus.nn.activation("Boxed", closes_over_a_list())


def test_number_closures_and_math_names_travel_in_the_archive(tmp_path):
    def scaled(k):
        def body(x):
            return x * k
        return body

    def tanh(x):
        return math.tanh(x)

    model = nexus.nn.Sequential()
    model.add(nexus.nn.activation("Times", scaled(2.0)))
    model.add(nexus.nn.activation("TanhPy", tanh))
    x = nexus.Tensor([1])
    x.copy_from([1.5])
    first = model.forward(x).to_list()
    assert abs(first[0] - math.tanh(3.0)) < 1e-5
    path = str(tmp_path / "closure.nxs")
    model.save_nxs(path)
    assert abs(nexus.load(path).forward(x).to_list()[0] - first[0]) < 1e-5
    r = _fresh_process(f"import nexus\nm = nexus.load({path!r})\nx = nexus.Tensor([1])\nx.copy_from([1.5])\n"
                       "print(m.forward(x).to_list()[0])\n")
    assert r.returncode == 0, r.stderr
    assert abs(float(r.stdout.strip()) - math.tanh(3.0)) < 1e-5


def _scale_forward(values, params):
    w = params[0].to_list()[0]
    out = type(values)(values.shape)
    out.copy_from([v * w for v in values.to_list()])
    return out


def _scale_backward(grad, params):
    w = params[0]["values"].to_list()[0]
    g = grad.to_list()
    params[0]["grad"].copy_from([sum(g)])
    out = type(grad)(grad.shape)
    out.copy_from([v * w for v in g])
    return out


def test_python_module_with_parameters_forward_backward_and_fresh_process(tmp_path):
    layer = nexus.nn.PythonModule("Scale", _scale_forward, _scale_backward, [[1]])
    layer.parameters()[0]["values"].copy_from([2.0])
    model = nexus.nn.Sequential()
    model.add(layer)
    x = nexus.Tensor([2])
    x.copy_from([1.5, -0.5])
    first = model.forward(x).to_list()
    assert abs(first[0] - 3.0) < 1e-5
    g = nexus.Tensor([2])
    g.copy_from([1.0, 1.0])
    back = model.backward(g).to_list()
    assert abs(back[0] - 2.0) < 1e-5
    assert abs(model.parameters()[0]["grad"].to_list()[0] - 2.0) < 1e-5
    path = str(tmp_path / "scale.nxs")
    model.save_nxs(path)
    assert max(abs(a - b) for a, b in zip(first, nexus.load(path).forward(x).to_list())) < 1e-5
    r = _fresh_process(f"import nexus\nm = nexus.load({path!r})\nx = nexus.Tensor([2])\nx.copy_from([1.5, -0.5])\n"
                       "print(m.forward(x).to_list())\n")
    assert r.returncode == 0, r.stderr
    assert "3.0" in r.stdout


# ------------------------------------------------------------------------------------------ tensors and images
def test_tensor_views_indexing_and_buffer_protocol():
    t = nexus.Tensor([6])
    t.copy_from([1, 2, 3, 4, 5, 6])
    view = t.reshape([2, 3])
    assert view.shape == [2, 3] and view[1, 2] == 6.0
    view[0, 1] = 9.0
    assert t[1] == 9.0
    mirror = memoryview(t)
    assert mirror.shape == (6,) and abs(mirror[1] - 9.0) < 1e-6


def test_images_write_read_convert_and_resize(tmp_path):
    chw = [1.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 1.0, 1.0]
    path = str(tmp_path / "square.png")
    nexus.data.save_image(path, chw, 2, 2, 3)
    back = nexus.data.load_image(path)
    assert (back["height"], back["width"], back["channels"]) == (2, 2, 3)
    assert abs(back["chw"][0] - 1.0) < 1e-6 and abs(back["chw"][1]) < 1e-6
    small = nexus.data.load_image(path, channels=3, height=1, width=1)
    assert (small["height"], small["width"]) == (1, 1) and len(small["chw"]) == 3
    grey = nexus.data.load_image(path, channels=1)
    assert grey["channels"] == 1 and len(grey["chw"]) == 4


def test_csv_tape_and_gemm(tmp_path):
    p = tmp_path / "rows.csv"
    p.write_text("1,0,1\n-1,0,0\n", encoding="utf-8")
    table = nexus.data.read_csv(str(p))
    assert table.features_per_sample == 2 and table.labels == [1, 0]
    tape = nexus.custom.MicroTape()
    x = tape.input(3.0)
    y = tape.square(x)
    tape.backward(y)
    assert abs(tape.value(y) - 9.0) < 1e-5 and abs(tape.grad(x) - 6.0) < 1e-4
    assert tape.size() == 2
    tape.reset()
    assert tape.size() == 0
    c = nexus.linalg.gemm(2, 2, 2, [1, 0, 0, 1], [2, 0, 0, 3])
    assert abs(c[0] - 2.0) < 1e-4 and abs(c[3] - 3.0) < 1e-4
    assert nexus.linalg.kernel_name()
    mean = nexus.train.all_reduce_mean([[1.0, 3.0], [3.0, 5.0]])
    assert abs(mean[0][0] - 2.0) < 1e-5 and abs(mean[1][1] - 4.0) < 1e-5


def test_tensor_tape_matches_a_finite_difference():
    first = nexus.nn.Linear(2, 2, True)
    second = nexus.nn.Linear(2, 1, True)
    first.parameters()[0]["values"].copy_from([0.2, 0.1, 0.0, 0.3])
    first.parameters()[1]["values"].copy_from([0.4, 0.5])
    second.parameters()[0]["values"].copy_from([0.3, -0.2])
    second.parameters()[1]["values"].copy_from([0.1])
    x = nexus.Tensor([1, 2])
    x.copy_from([0.5, -0.25])
    tape = nexus.custom.Tape()
    hidden = tape.apply(first, tape.input(x))
    out = tape.apply(second, tape.relu(hidden))
    first.zero_grad()
    second.zero_grad()
    tape.backward(out)
    analytic = first.parameters()[0]["grad"].to_list()[0]
    weight = first.parameters()[0]["values"]
    base = weight.to_list()

    def score(delta):
        changed = list(base)
        changed[0] += delta
        weight.copy_from(changed)
        return second.forward(nexus.nn.ReLU().forward(first.forward(x))).to_list()[0]

    numeric = (score(1e-3) - score(-1e-3)) / 2e-3
    assert abs(analytic - numeric) < 1e-4


def test_convolutions():
    out = nexus.nn.conv2d_device([2.0], [3.0], [0.5], 1, 1, 1, 1, 1, 1, 1, 1, 0)
    assert out["height"] == 1 and out["width"] == 1 and abs(out["nchw"][0] - 6.5) < 1e-4
    layer = nexus.nn.Conv2d(1, 1, 1, 1, 0, True)
    image = nexus.Tensor([1, 1, 1, 1])
    image.copy_from([1.0])
    assert layer.forward(image).numel() == 1


# -------------------------------------------------------------------------------------------------------- rl
def test_agents_buffers_league_and_vector_env(tmp_path):
    env = nexus.rl.LineWorld()
    cfg = nexus.rl.PPOConfig()
    cfg.hidden, cfg.seed, cfg.epochs = 8, 2, 1
    agent = nexus.rl.PPOAgent(env.observation_dim(), env.action_count(), cfg)
    agent.learn(env, 1, 4)
    obs = [0.0] * env.observation_dim()
    action = agent.act(obs, True)[0]
    path = str(tmp_path / "agent.nxs")
    agent.save_nxs(path)
    assert nexus.rl.PPOAgent.load_nxs(path).act(obs, True)[0] == action
    league = nexus.rl.League()
    pid = league.add_player(1200.0)
    league.save(pid, [0.5, 0.25])
    lpath = str(tmp_path / "league.nxs")
    league.save_nxs(lpath)
    back = nexus.rl.League.load_nxs(lpath)
    assert abs(back.elo(0) - 1200.0) < 1e-3 and back.weights(0) == [0.5, 0.25]
    venv = nexus.rl.VectorEnv.line_worlds(2)
    assert len(venv.reset(1)) == 2 * nexus.rl.LineWorld().observation_dim()
    assert len(venv.step([0, 1])["rewards"]) == 2

    buf = nexus.rl.ReplayBuffer(4, 2)
    buf.add([0.0, 1.0], 1, 0.5, [1.0, 0.0], False)
    s = buf.sample([0])
    assert s["actions"] == [1] and abs(s["rewards"][0] - 0.5) < 1e-6
    per = nexus.rl.PrioritizedReplayBuffer(4, 2, 0.6)
    per.add([0.0, 1.0], 0, 1.0, [1.0, 0.0], False, 1.0)
    assert per.sample(1, 0.4, 3)["actions"] == [0]
    roll = nexus.rl.RolloutBuffer()
    roll.reset(1, 2)
    roll.add([0.2, 0.3], 1, -0.1, 0.4, 1.0, False)
    roll.finish(0.99, 0.95, 0.0)
    assert roll.size() == 1 and roll.actions()[0] == 1
    ac = nexus.rl.ActorCriticAgent.discrete(2, 2, 1)
    a, logp, value = ac.act([0.0, 1.0], True)
    assert a in (0, 1) and isinstance(logp, float) and isinstance(value, float)
    cont = nexus.rl.ContinuousActorCritic(1, 1)
    assert -1.0 <= cont.act([0.25], True) <= 1.0


def test_python_environment_subclass():
    class Counter(nexus.rl.Environment):
        def __init__(self):
            super().__init__(1, 2, True)
            self.value = 0.0

        def reset(self, seed):
            self.value = 0.0
            return [self.value]

        def step(self, action):
            self.value = 1.0 if int(action) == 1 else 0.0
            return {"observation": [self.value], "reward": float(action), "terminated": False, "truncated": False,
                    "info": "py"}

    env = Counter()
    assert env.reset(1) == [0.0]
    st = env.step(1)
    assert st["observation"] == [1.0] and st["reward"] == 1.0 and st["info"] == "py"
    assert env.observation_dim() == 1 and env.action_count() == 2


# ------------------------------------------------------------------------------------------ graph + small LM
def _identity(layer, width):
    w = [0.0] * (width * width)
    for i in range(width):
        w[i * width + i] = 1.0
    layer.parameters()[0]["values"].copy_from(w)
    if len(layer.parameters()) > 1:
        b = layer.parameters()[1]["values"]
        b.copy_from([0.0] * b.numel())


def test_graph_concatenates_two_named_nodes():
    left, right, joined = nexus.nn.Linear(2, 2, True), nexus.nn.Linear(2, 2, True), nexus.nn.Linear(4, 4, True)
    _identity(left, 2)
    _identity(right, 2)
    _identity(joined, 4)
    g = nexus.nn.Graph()
    g.add("n2", left)
    g.add("n3", nexus.nn.ReLU())
    g.add("n4", right)
    g.concat("n5", joined, ["n4", "n2"])
    x = nexus.Tensor([1, 2])
    x[0], x[1] = 3.0, 5.0
    out = g.forward(x).to_list()
    assert len(out) == 4
    for got, want in zip(out, (3.0, 5.0, 3.0, 5.0)):
        assert abs(got - want) < 1e-5


def test_small_language_model_loss_drops():
    vocab, embed = 6, 8
    model = nexus.nn.Sequential()
    model.add(nexus.nn.Embedding(vocab, embed, -1))
    model.add(nexus.nn.PositionalEncoding(embed, 32, False))
    model.add(nexus.nn.CausalTransformerBlock(embed, 2, 16))
    model.add(nexus.nn.Linear(embed, vocab, True))
    trainer = nexus.train.LanguageTrainer(model, 0.08)
    rows = [[t % vocab for t in range(8)] for _ in range(4)]
    first = trainer.fit(rows, 1)
    later = trainer.fit(rows, 30)
    assert later < first
