"""Graph passes: dead-code elimination, constant folding, common-subexpression elimination, the seven
rewrite patterns (selected by a bit mask), the joint forward+backward graph (reverse-mode AD on the IR),
element-wise fusion (vertical chains and horizontal siblings), min-cut recomputation (max-flow over the
activation graph), static memory planning and communication scheduling.
Parity: include/nexus/compile/passes.hpp:25-90, src/compile/passes.cpp of the reference."""
from __future__ import annotations

from collections import deque
from typing import Dict, List, Optional, Set, Tuple

from .ir import COMM, ELEMENTWISE, Graph, Node, Value

P_LINEAR_BIAS_GELU, P_ADD_NORM, P_ATTENTION_QKV, P_GATED, P_LINEAR_CE, P_LINEAR_BIAS, P_IDENTITY = 1, 2, 4, 8, 16, 32, 64
P_ALL = 127


def _replace_uses(g: Graph, old: Value, new: Value) -> None:
    for n in g.nodes:
        n.inputs = [new if v is old else v for v in n.inputs]
    g.outputs = [new if v is old else v for v in g.outputs]


def toposort(g: Graph) -> None:
    """Stable topological order (a rewrite may make a node read a value defined later in the list)."""
    placed: Set[int] = set()
    order: List[Node] = []
    pending = list(g.nodes)
    while pending:
        rest = []
        for n in pending:
            if all(v.producer is None or id(v.producer) in placed for v in n.inputs):
                order.append(n)
                placed.add(id(n))
            else:
                rest.append(n)
        if len(rest) == len(pending):
            raise ValueError("graph has a cycle")
        pending = rest
    g.nodes = order


def dce(g: Graph) -> int:
    live: Set[int] = set()
    work = [v for v in g.outputs]
    while work:
        v = work.pop()
        n = v.producer
        if n is None or id(n) in live:
            continue
        live.add(id(n))
        work.extend(n.inputs)
    before = len(g.nodes)
    g.nodes = [n for n in g.nodes if id(n) in live or n.op in COMM and n.attrs.get("side_effect")]
    g.params = {k: v for k, v in g.params.items() if v.producer is not None and id(v.producer) in live}
    g.inputs = [v for v in g.inputs if id(v.producer) in live]
    return before - len(g.nodes)


def cse(g: Graph) -> int:
    seen: Dict[tuple, Node] = {}
    removed = 0
    for n in list(g.nodes):
        if n.op in ("Param", "Input") or n.op in COMM:
            continue
        key = (n.op, tuple(v.id for v in n.inputs), Graph._attr_s(n.attrs))
        if key in seen:
            for old, new in zip(n.outputs, seen[key].outputs):
                _replace_uses(g, old, new)
            g.nodes.remove(n)
            removed += 1
        else:
            seen[key] = n
    return removed


def constant_fold(g: Graph) -> int:
    """Scale(Scale(x, a), b) -> Scale(x, a*b); Scale(Const c, a) -> Const(c*a); Add / Mul of two constants."""
    changed = 0
    for n in list(g.nodes):
        if n.op == "Scale" and n.inputs[0].producer is not None:
            p = n.inputs[0].producer
            if p.op == "Scale":
                n.attrs["factor"] = float(n.attrs["factor"]) * float(p.attrs["factor"])
                n.inputs = [p.inputs[0]]
                changed += 1
            elif p.op == "Const":
                n.op, n.inputs = "Const", []
                n.attrs = {"value": float(p.attrs["value"]) * float(n.attrs["factor"])}
                changed += 1
        elif n.op in ("Add", "Mul") and all(v.producer is not None and v.producer.op == "Const" for v in n.inputs):
            a, b = (float(v.producer.attrs["value"]) for v in n.inputs)
            n.attrs = {"value": a + b if n.op == "Add" else a * b}
            n.op, n.inputs = "Const", []
            changed += 1
    if changed:
        dce(g)
    return changed


def _single_user(users, v: Value) -> Optional[Node]:
    u = users.get(v, [])
    return u[0] if len(u) == 1 else None


def rewrite_patterns(g: Graph, mask: int = P_ALL) -> Dict[str, int]:
    stats = {"linear_bias_gelu": 0, "add_norm": 0, "attention_qkv": 0, "gated": 0, "linear_ce": 0, "linear_bias": 0,
             "identity": 0}
    users = g.users()

    def refresh():
        nonlocal users
        users = g.users()

    if mask & P_IDENTITY:
        for n in list(g.nodes):
            if (n.op == "Scale" and float(n.attrs.get("factor", 0)) == 1.0) or \
               (n.op == "Reshape" and n.inputs[0].shape == n.outputs[0].shape):
                _replace_uses(g, n.outputs[0], n.inputs[0])
                g.nodes.remove(n)
                stats["identity"] += 1
        refresh()
    if mask & (P_LINEAR_BIAS_GELU | P_LINEAR_BIAS):
        for n in list(g.nodes):
            if n.op != "Linear" or len(n.inputs) != 2:
                continue
            b = _single_user(users, n.outputs[0])
            if b is None or b.op != "Bias":
                continue
            act = _single_user(users, b.outputs[0])
            if (mask & P_LINEAR_BIAS_GELU) and act is not None and act.op == "Gelu":
                n.op, n.inputs, n.outputs = "LinearBiasGelu", [n.inputs[0], n.inputs[1], b.inputs[1]], act.outputs
                act.outputs[0].producer = n
                g.nodes.remove(b)
                g.nodes.remove(act)
                stats["linear_bias_gelu"] += 1
            elif mask & P_LINEAR_BIAS:
                n.inputs, n.outputs = [n.inputs[0], n.inputs[1], b.inputs[1]], b.outputs
                n.attrs["has_bias"] = True
                b.outputs[0].producer = n
                g.nodes.remove(b)
                stats["linear_bias"] += 1
            refresh()
    if mask & P_ATTENTION_QKV:
        for n in list(g.nodes):
            if n.op != "SplitQKV":
                continue
            us = [_single_user(users, o) for o in n.outputs]
            if us[0] is not None and us[0].op == "Attention" and all(u is us[0] for u in us):
                att = us[0]
                att.op, att.inputs = "AttentionQKV", [n.inputs[0]]
                att.attrs.update(n.attrs)
                g.nodes.remove(n)
                stats["attention_qkv"] += 1
                refresh()
    if mask & P_GATED:
        for n in list(g.nodes):
            if n.op != "GatedSplit":
                continue
            act = _single_user(users, n.outputs[0])
            mul = _single_user(users, n.outputs[1])
            if act is None or mul is None or act.op not in ("Silu", "Gelu") or mul.op != "Mul":
                continue
            if _single_user(users, act.outputs[0]) is not mul:
                continue
            mul.op, mul.inputs = ("SwiGlu" if act.op == "Silu" else "GeGlu"), [n.inputs[0]]
            g.nodes.remove(n)
            g.nodes.remove(act)
            stats["gated"] += 1
            refresh()
    if mask & P_ADD_NORM:
        for n in list(g.nodes):
            if n.op != "Add":
                continue
            norms = [u for u in users.get(n.outputs[0], []) if u.op in ("LayerNorm", "RmsNorm") and u.inputs[0] is n.outputs[0]]
            if len(norms) != 1:
                continue
            nm = norms[0]
            # AddNorm(a, b, gamma[, beta]) -> (sum, normed); the sum stays available to the residual stream
            n.op = "AddNorm"
            n.attrs = {"kind": nm.op, "eps": nm.attrs.get("eps", 1e-5)}
            n.inputs = n.inputs + nm.inputs[1:]
            n.outputs = [n.outputs[0], nm.outputs[0]]
            nm.outputs[0].producer = n
            g.nodes.remove(nm)
            stats["add_norm"] += 1
            refresh()
    if mask & P_LINEAR_CE:
        for n in list(g.nodes):
            if n.op != "CrossEntropyShifted":
                continue
            lin = n.inputs[0].producer
            if lin is not None and lin.op == "Linear" and len(lin.inputs) == 2 and _single_user(users, lin.outputs[0]) is n:
                n.op, n.inputs = "FusedLinearCE", [lin.inputs[0], lin.inputs[1], n.inputs[1]]
                g.nodes.remove(lin)
                stats["linear_ce"] += 1
                refresh()
    toposort(g)
    return stats


# ---------------------------------------------------------------------------------------- joint graph
NON_DIFF_INPUT = {("Embedding", 0), ("CrossEntropyShifted", 1), ("FusedLinearCE", 2)}


def build_joint(g: Graph) -> Tuple[Graph, Dict[str, Value]]:
    """Appends the backward pass to (a copy-free view of) ``g``: one ``Vjp`` node per forward node in reverse
    order, ``Accumulate`` nodes where a value has several users.  Returns (graph, {param name: grad value})."""
    if len(g.outputs) != 1:
        raise ValueError("build_joint expects a single scalar output")
    fwd_nodes = list(g.nodes)
    grads: Dict[Value, Value] = {}
    (seed,) = g.add("Const", [], [[]], value=1.0)
    grads[g.outputs[0]] = seed
    for idx in range(len(fwd_nodes) - 1, -1, -1):
        n = fwd_nodes[idx]
        if n.op in ("Param", "Input", "Const"):
            continue
        gouts = [grads.get(o) for o in n.outputs]
        if all(x is None for x in gouts):
            continue
        diff = [i for i, v in enumerate(n.inputs) if (n.op, i) not in NON_DIFF_INPUT and v.dtype == "f32"]
        if not diff:
            continue
        present = [x for x in gouts if x is not None]
        outs = g.add("Vjp", list(n.inputs) + list(n.outputs) + present, [n.inputs[i].shape for i in diff],
                     fwd=n, fwd_op=n.op, wrt=diff, have=[i for i, x in enumerate(gouts) if x is not None])
        for i, gv in zip(diff, outs):
            v = n.inputs[i]
            if v in grads:
                (grads[v],) = g.add("Accumulate", [grads[v], gv], [v.shape])
            else:
                grads[v] = gv
    pgrads = {name: grads[v] for name, v in g.params.items() if v in grads}
    g.outputs = [g.outputs[0]] + list(pgrads.values())
    return g, pgrads


def fuse_epilogues(g: Graph) -> Dict[str, int]:
    """Folds what a GEMM epilogue can do into the backward nodes of a joint graph.

    * ``beta1``: ``Accumulate(a, b)`` whose ``b`` is the only use of a ``Vjp`` output disappears; the ``Vjp`` node
      takes ``a`` as an extra input and adds its result onto it (the weight-gradient GEMM run with beta = 1, the
      residual-stream gradient added in the input-gradient GEMM's epilogue), so no separate add and no temporary.
    * ``dgelu`` / ``bgrad``: the ``Vjp`` of a ``LinearBiasGelu`` node is marked as one fused backward (GELU derivative
      in the input-gradient epilogue, bias gradient as the column sum taken with the weight gradient); the ``Vjp`` of a
      ``Bias`` that follows a ``Linear`` is marked ``bgrad`` with the linear's ``Vjp`` it rides on.
    Returns the number of each.  Values and results are unchanged; only nodes and temporaries go away.
    Parity: ``fuse_epilogues`` (DGELU / BGRAD / beta = 1) of include/nexus/compile/passes.hpp in the reference."""
    counts = {"beta1": 0, "dgelu": 0, "bgrad": 0}
    users = g.users()
    pos = {id(n): i for i, n in enumerate(g.nodes)}
    drop = set()
    for n in list(g.nodes):
        if n.op != "Accumulate" or len(n.inputs) != 2:
            continue
        a, b = n.inputs
        prod = b.producer
        if prod is None or prod.op != "Vjp" or len(users.get(b, [])) != 1:
            a, b = b, a                                   # the Vjp result may sit on either side
            prod = b.producer
            if prod is None or prod.op != "Vjp" or len(users.get(b, [])) != 1:
                continue
        if a.producer is not None and pos[id(a.producer)] > pos[id(prod)]:
            continue                                      # the running sum must exist before the Vjp runs
        if b in g.outputs:
            continue
        k = prod.outputs.index(b)
        acc = dict(prod.attrs.get("accumulate", {}))
        if k in acc:
            continue
        acc[k] = len(prod.inputs)                         # position of the running sum among the node's inputs
        prod.attrs["accumulate"] = acc
        prod.inputs.append(a)
        _replace_uses(g, n.outputs[0], b)
        g.outputs = [b if v is n.outputs[0] else v for v in g.outputs]
        b.shape, b.name = n.outputs[0].shape, n.outputs[0].name or b.name
        drop.add(id(n))
        counts["beta1"] += 1
    if drop:
        g.nodes = [n for n in g.nodes if id(n) not in drop]
    vjp_of = {id(n.attrs["fwd"]): n for n in g.nodes if n.op == "Vjp"}
    for n in g.nodes:
        if n.op != "Vjp":
            continue
        f = n.attrs["fwd"]
        if f.op == "LinearBiasGelu":
            n.attrs["epilogue"] = "dgelu+bgrad"
            counts["dgelu"] += 1
            counts["bgrad"] += 1
        elif f.op == "Bias" and f.inputs and f.inputs[0].producer is not None and f.inputs[0].producer.op == "Linear":
            lin = vjp_of.get(id(f.inputs[0].producer))
            if lin is not None:
                n.attrs["epilogue"] = "bgrad"
                lin.attrs["epilogue"] = "bgrad"
                counts["bgrad"] += 1
    return counts


# ---------------------------------------------------------------------------------------- fusion
def fuse_elementwise(g: Graph) -> Dict[str, int]:
    """Vertical: a chain of element-wise nodes whose intermediate values have a single user becomes one
    ``Fused`` node (body = the chain).  Horizontal: element-wise siblings reading the same value with the same
    shape become one multi-output ``Fused`` node."""
    stats = {"vertical": 0, "horizontal": 0}
    users = g.users()
    done: Set[int] = set()
    for n in list(g.nodes):
        if n.op not in ELEMENTWISE or id(n) in done or n not in g.nodes:
            continue
        chain = [n]
        cur = n
        while True:
            nxt = _single_user(users, cur.outputs[0])
            if nxt is None or nxt.op not in ELEMENTWISE or nxt.outputs[0].shape != cur.outputs[0].shape:
                break
            chain.append(nxt)
            cur = nxt
        if len(chain) < 2:
            continue
        internal = {c.outputs[0] for c in chain[:-1]}
        ext: List[Value] = []
        for c in chain:
            for v in c.inputs:
                if v not in internal and v not in ext:
                    ext.append(v)
        body = [(c.op, dict(c.attrs), [(("in", ext.index(v)) if v in ext else ("tmp", [k.outputs[0] for k in chain].index(v)))
                                       for v in c.inputs]) for c in chain]
        pos = g.nodes.index(chain[-1])
        fused = Node("Fused", ext, chain[-1].outputs, {"body": body, "kind": "vertical"})
        chain[-1].outputs[0].producer = fused
        g.nodes[pos] = fused
        for c in chain[:-1]:
            g.nodes.remove(c)
            done.add(id(c))
        done.add(id(chain[-1]))
        stats["vertical"] += 1
        users = g.users()
    users = g.users()
    for v, us in list(users.items()):
        sib = [u for u in us if u.op in ELEMENTWISE and len(u.inputs) == 1 and u in g.nodes]
        if len(sib) >= 2:
            body = [(u.op, dict(u.attrs), [("in", 0)]) for u in sib]
            pos = min(g.nodes.index(u) for u in sib)
            fused = Node("Fused", [v], [u.outputs[0] for u in sib], {"body": body, "kind": "horizontal"})
            for u in sib:
                u.outputs[0].producer = fused
                g.nodes.remove(u)
            g.nodes.insert(pos, fused)
            stats["horizontal"] += 1
    return stats


# ---------------------------------------------------------------------------------------- min cut
class _Dinic:
    def __init__(self, n: int):
        self.n, self.adj = n, [[] for _ in range(n)]

    def edge(self, u: int, v: int, c: float) -> None:
        self.adj[u].append([v, c, len(self.adj[v])])
        self.adj[v].append([u, 0.0, len(self.adj[u]) - 1])

    def flow(self, s: int, t: int) -> float:
        total = 0.0
        while True:
            level = [-1] * self.n
            level[s] = 0
            q = deque([s])
            while q:
                u = q.popleft()
                for v, c, _ in self.adj[u]:
                    if c > 1e-12 and level[v] < 0:
                        level[v] = level[u] + 1
                        q.append(v)
            if level[t] < 0:
                return total
            it = [0] * self.n

            def dfs(u, f):
                if u == t:
                    return f
                while it[u] < len(self.adj[u]):
                    e = self.adj[u][it[u]]
                    v, c, r = e
                    if c > 1e-12 and level[v] == level[u] + 1:
                        d = dfs(v, min(f, c))
                        if d > 0:
                            e[1] -= d
                            self.adj[v][r][1] += d
                            return d
                    it[u] += 1
                return 0.0
            while True:
                f = dfs(s, float("inf"))
                if f <= 0:
                    break
                total += f

    def source_side(self, s: int) -> Set[int]:
        seen, q = {s}, deque([s])
        while q:
            u = q.popleft()
            for v, c, _ in self.adj[u]:
                if c > 1e-12 and v not in seen:
                    seen.add(v)
                    q.append(v)
        return seen


CHEAP = ELEMENTWISE | {"LayerNorm", "RmsNorm", "Bias", "GatedSplit", "SplitQKV", "Rope", "SwiGlu", "GeGlu", "Fused", "Reshape"}


def min_cut_recompute(g: Graph, env: Dict[str, int]) -> Dict[str, object]:
    """Chooses which forward values to keep for the backward pass.  Values needed by ``Vjp`` nodes are the
    sinks; a value may be recomputed from its inputs when its producer is cheap (element-wise, norms,
    splits), so the minimum cut of the forward value graph (capacities = bytes) is the cheapest set to save."""
    fwd = [n for n in g.nodes if n.op not in ("Vjp", "Accumulate")]
    needed: Set[Value] = set()
    for n in g.nodes:
        if n.op == "Vjp":
            f: Node = n.attrs["fwd"]
            needed.update(v for v in list(f.inputs) + list(f.outputs) if v.dtype == "f32" and v.producer is not None
                          and v.producer.op not in ("Param", "Input", "Const"))
    vals = [o for n in fwd for o in n.outputs if n.op not in ("Param", "Input", "Const")]
    idx = {v: i for i, v in enumerate(vals)}
    S, Tn = 2 * len(vals), 2 * len(vals) + 1
    net = _Dinic(2 * len(vals) + 2)
    INF = float("inf")
    for v in vals:
        i = idx[v]
        net.edge(2 * i, 2 * i + 1, float(v.numel(env) * 4))       # cutting here = saving v
        p = v.producer
        if p.op in CHEAP:
            srcs = [u for u in p.inputs if u in idx]
            for u in srcs:
                net.edge(2 * idx[u] + 1, 2 * i, INF)
            if not srcs:
                net.edge(S, 2 * i, INF)                           # recomputable from parameters / inputs alone
        else:
            net.edge(S, 2 * i, INF)                               # expensive producer: only available by saving
        if v in needed:
            net.edge(2 * i + 1, Tn, INF)
    total_needed = sum(v.numel(env) * 4 for v in needed)
    cut = net.flow(S, Tn)
    side = net.source_side(S)
    saved = [v for v in vals if 2 * idx[v] in side and 2 * idx[v] + 1 not in side]
    recomputed = [v for v in needed if v not in saved]
    for v in recomputed:
        v.producer.attrs["recompute"] = True
    return {"saved": saved, "recomputed": recomputed, "saved_bytes": int(cut), "baseline_bytes": int(total_needed)}


# ---------------------------------------------------------------------------------------- memory / comm
def plan_memory(g: Graph, env: Dict[str, int], alignment: int = 256) -> Dict[str, object]:
    """Static arena for every non-parameter value from its lifetime (definition .. last use)."""
    from .. import _native
    first, last = {}, {}
    for i, n in enumerate(g.nodes):
        for o in n.outputs:
            first[o] = i
            last[o] = i
        for v in n.inputs:
            last[v] = i
    for v in g.outputs:
        last[v] = len(g.nodes)
    vals = [v for v in first if v.producer.op not in ("Param", "Input")]
    life = [(max(4, v.numel(env) * 4), first[v], last[v]) for v in vals]
    offsets, arena = _native.plan_memory(life, alignment)
    naive = sum(-(-b // alignment) * alignment for b, _, _ in life)
    return {"offsets": {v.id: o for v, o in zip(vals, offsets)}, "arena_bytes": int(arena), "naive_bytes": int(naive)}


def schedule_communication(g: Graph) -> int:
    """Moves every gather-type communication node as early as its inputs allow (prefetch) and marks where its
    result is first needed, so that an executor can issue it asynchronously and wait just before the consumer."""
    moved = 0
    for n in list(g.nodes):
        if n.op not in COMM:
            continue
        pos = g.nodes.index(n)
        ready = 0
        for v in n.inputs:
            if v.producer is not None:
                ready = max(ready, g.nodes.index(v.producer) + 1)
        if n.op in ("AllGather", "Recv") and ready < pos:
            g.nodes.remove(n)
            g.nodes.insert(ready, n)
            moved += 1
        users = [i for i, m in enumerate(g.nodes) if any(v in n.outputs for v in m.inputs)]
        n.attrs["async"] = True
        n.attrs["wait_before"] = min(users) if users else len(g.nodes)
    return moved
