"""Seeded synthetic SPNs and input batches for the benchmark configurations.

Every generator returns a `FlatSPN` (flat arrays, children before parents) that
`to_xspn_bytes()` turns into a regular xspn query file, i.e. the engine is fed exactly what a
user of `CUDACompiler` would feed it.  Structures follow a LearnSPN-like recursion: a sum node
mixes `fan-in` product nodes, a product node splits its scope into random parts, each part is
modelled by a sum node again, and the recursion ends in products of univariate leaves.
The shapes echo public data sets only in their dimensions; all values are drawn from
`numpy.random.default_rng(seed)`.
"""
import numpy as np

from xspn.serialization.binary import wire


class FlatSPN:
    def __init__(self, num_features, feature_type, name):
        self.F = num_features
        self.feature_type = feature_type
        self.name = name
        self.kind, self.scope_id, self.mean, self.stddev = [], [], [], []
        self.child_ptr, self.tab_ptr, self.brk_ptr = [0], [0], [0]
        self.child_id, self.weight, self.tab, self.brk = [], [], [], []
        self.root = -1

    def _add(self, kind, children=(), weights=(), scope=0, mean=0.0, stddev=1.0, tab=(), brk=()):
        self.kind.append(kind)
        self.scope_id.append(scope)
        self.mean.append(mean)
        self.stddev.append(stddev)
        self.child_id.extend(children)
        self.weight.extend(weights if len(weights) else [0.0] * len(children))
        self.tab.extend(tab)
        self.brk.extend(brk)
        self.child_ptr.append(len(self.child_id))
        self.tab_ptr.append(len(self.tab))
        self.brk_ptr.append(len(self.brk))
        return len(self.kind) - 1

    def gaussian(self, f, mean, stddev):
        return self._add(wire.K_GAUSS, scope=f, mean=float(mean), stddev=float(stddev))

    def categorical(self, f, p):
        return self._add(wire.K_CAT, scope=f, tab=[float(v) for v in p])

    def histogram(self, f, breaks, dens):
        return self._add(wire.K_HIST, scope=f, tab=[float(v) for v in dens], brk=[int(b) for b in breaks])

    def product(self, children):
        return self._add(wire.K_PRODUCT, children=list(children))

    def sum(self, children, weights):
        return self._add(wire.K_SUM, children=list(children), weights=[float(w) for w in weights])

    @property
    def num_nodes(self):
        return len(self.kind)

    def stats(self):
        k = np.asarray(self.kind)
        return {"nodes": len(k), "sums": int((k == wire.K_SUM).sum()), "products": int((k == wire.K_PRODUCT).sum()),
                "leaves": int((k >= wire.K_HIST).sum()), "edges": len(self.child_id)}

    def to_xspn_bytes(self, batch_size=64, support_marginal=True, error_kind=0, max_error=0.02):
        n = len(self.kind)
        return wire.encode_flat(
            kind=self.kind, node_id=np.arange(n), child_ptr=self.child_ptr, child_id=np.asarray(self.child_id, np.int32),
            weight=np.asarray(self.weight, np.float64), scope_id=self.scope_id, mean=self.mean, stddev=self.stddev,
            tab_ptr=self.tab_ptr, tab=np.asarray(self.tab, np.float64), brk_ptr=self.brk_ptr,
            brk=np.asarray(self.brk, np.int32), root_id=self.root, scope=list(range(self.F)),
            feature_type=self.feature_type, name=self.name,
            query={"batch_size": batch_size, "error_kind": error_kind, "max_error": max_error,
                   "support_marginal": support_marginal})


def _dirichlet(rng, k):
    w = rng.dirichlet(np.ones(k))
    w = np.maximum(w, 1e-6)
    return w / w.sum()


class _Builder:
    """Budgeted LearnSPN-like recursion.  `leaf(f)` creates one univariate leaf on feature f."""

    def __init__(self, spn, rng, leaf, fanin, parts, share=0.0):
        self.spn, self.rng, self.leaf = spn, rng, leaf
        self.fanin, self.parts, self.share = fanin, parts, share
        self.pool = {}        # scope -> product nodes usable by other sums over the same scope
        self.part_cache = {}  # scope -> fixed partition (only when sharing, so that scopes recur)

    def sum_node(self, scope, layers, budget):
        """`layers` = sum/product layers still allowed below and including this sum."""
        k = int(self.rng.integers(self.fanin[0], self.fanin[1] + 1))
        # keep enough budget per child for the recursion to reach the requested depth
        k = max(self.fanin[0], min(k, budget // (3 * len(scope) + 4)))
        kids = []
        pool = self.pool.setdefault(scope, []) if self.share > 0 else None
        for _ in range(k):
            if pool and self.rng.random() < self.share:
                cand = pool[int(self.rng.integers(len(pool)))]
                if cand not in kids:
                    kids.append(cand)
                    continue
            p = self.product_node(scope, layers - 1, max((budget - 1) // k, 1))
            if pool is not None:
                pool.append(p)
            kids.append(p)
        return self.spn.sum(kids, _dirichlet(self.rng, len(kids)))

    def product_node(self, scope, layers, budget):
        nvar = len(scope)
        if layers <= 1 or nvar == 1 or budget < 2 * nvar + 4:
            return self.spn.product([self.leaf(f) for f in scope])
        if self.share > 0 and scope in self.part_cache:
            parts = self.part_cache[scope]
        else:
            p = int(min(self.rng.integers(self.parts[0], self.parts[1] + 1), nvar))
            perm = self.rng.permutation(nvar)
            cuts = np.sort(self.rng.choice(np.arange(1, nvar), size=p - 1, replace=False)) if p > 1 else []
            parts = [tuple(sorted(scope[i] for i in seg)) for seg in np.split(perm, cuts)]
            if self.share > 0:
                self.part_cache[scope] = parts
        kids = []
        for part in parts:
            b = max((budget - 1) * len(part) // nvar, 1)
            if len(part) == 1:
                kids.append(self.leaf(part[0]))
            else:
                kids.append(self.sum_node(part, layers - 1, b))
        return self.spn.product(kids)


def _grow(make, target, tol=0.12, tries=40):
    """Re-run the budgeted generator with a scaled budget until the node count is near target."""
    budget = target
    best = None
    for _ in range(tries):
        spn = make(int(budget))
        n = spn.num_nodes
        if best is None or abs(n - target) < abs(best.num_nodes - target):
            best = spn
        if abs(n - target) <= tol * target:
            break
        budget = max(budget * target / max(n, 1), 8)
    return best


# --------------------------------------------------------------------------------------------
# the five configurations
# --------------------------------------------------------------------------------------------
def config1(seed=1001, target_nodes=400):
    """16 categorical features (2-3 categories), depth 6, ~400 nodes, sum fan-in 2-4; int32 inputs."""
    def make(budget):
        rng = np.random.default_rng(seed)
        spn = FlatSPN(16, "int32", "cfg1_categorical")
        ncat = rng.integers(2, 4, size=16)
        spn.ncat = ncat
        b = _Builder(spn, rng, lambda f: spn.categorical(f, _dirichlet(rng, int(ncat[f]))), (2, 4), (2, 3))
        spn.root = b.sum_node(tuple(range(16)), 6, budget)
        return spn
    return _grow(make, target_nodes)


def config1_inputs(spn, n, seed=2001):
    rng = np.random.default_rng(seed)
    return (rng.integers(0, 1 << 30, size=(n, 16)) % spn.ncat[None, :]).astype(np.int32)


def config2(seed=1002, target_nodes=2000):
    """26 Gaussian features (mean~N(0,1), stddev~U(0.5,2)), depth 8, ~2000 nodes, fan-in 2-8."""
    def make(budget):
        rng = np.random.default_rng(seed)
        spn = FlatSPN(26, "float32", "cfg2_gaussian")
        b = _Builder(spn, rng, lambda f: spn.gaussian(f, rng.normal(), rng.uniform(0.5, 2.0)), (2, 8), (2, 3))
        spn.root = b.sum_node(tuple(range(26)), 8, budget)
        return spn
    return _grow(make, target_nodes)


def config2_inputs(n, seed=2002):
    return np.random.default_rng(seed).standard_normal((n, 26), dtype=np.float32)


def config3(seed=1003, target_nodes=8000):
    """100 integer features, Histogram leaves (4-16 near-equal-width buckets on [0,256)), depth 10."""
    def leaf_factory(spn, rng):
        def leaf(f):
            nb = int(rng.integers(4, 17))
            breaks = np.round(np.linspace(0, 256, nb + 1)).astype(int)
            return spn.histogram(f, breaks, _dirichlet(rng, nb))
        return leaf

    def make(budget):
        rng = np.random.default_rng(seed)
        spn = FlatSPN(100, "float32", "cfg3_histogram")
        b = _Builder(spn, rng, leaf_factory(spn, rng), (2, 4), (2, 4))
        spn.root = b.sum_node(tuple(range(100)), 10, budget)
        return spn
    return _grow(make, target_nodes)


def config3_inputs(n, seed=2003, nan_frac=0.10):
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 256, size=(n, 100)).astype(np.float32)
    x[rng.random((n, 100)) < nan_frac] = np.nan
    return x


def config4(seed=1004, target_nodes=50000):
    """256 mixed features (0..127 Gaussian, 128..255 Categorical K=4), depth 16, ~50k nodes, 20 % of
    product children re-used across the sums of one scope."""
    def make(budget):
        rng = np.random.default_rng(seed)
        spn = FlatSPN(256, "float32", "cfg4_mixed")

        def leaf(f):
            if f < 128:
                return spn.gaussian(f, rng.normal(), rng.uniform(0.5, 2.0))
            return spn.categorical(f, _dirichlet(rng, 4))
        b = _Builder(spn, rng, leaf, (2, 4), (2, 3), share=0.2)
        spn.root = b.sum_node(tuple(range(256)), 16, budget)
        return spn
    return _grow(make, target_nodes)


def config4_inputs(n, seed=2004):
    rng = np.random.default_rng(seed)
    x = np.empty((n, 256), np.float32)
    x[:, :128] = rng.standard_normal((n, 128), dtype=np.float32)
    x[:, 128:] = rng.integers(0, 4, size=(n, 128)).astype(np.float32)
    return x


class ArraySPN:
    """A model held as numpy arrays (for generators that are vectorised end to end)."""

    def __init__(self, num_features, feature_type, name, arrays, root):
        self.F, self.feature_type, self.name, self.a, self.root = num_features, feature_type, name, arrays, root

    @property
    def num_nodes(self):
        return len(self.a["kind"])

    def stats(self):
        k = self.a["kind"]
        return {"nodes": len(k), "sums": int((k == wire.K_SUM).sum()), "products": int((k == wire.K_PRODUCT).sum()),
                "leaves": int((k >= wire.K_HIST).sum()), "edges": len(self.a["child_id"])}

    def to_xspn_bytes(self, batch_size=64, support_marginal=True, error_kind=0, max_error=0.02):
        a = self.a
        n = len(a["kind"])
        z = np.zeros(n + 1, np.int64)
        return wire.encode_flat(
            kind=a["kind"], node_id=np.arange(n), child_ptr=a["child_ptr"], child_id=a["child_id"], weight=a["weight"],
            scope_id=a["scope_id"], mean=a["mean"], stddev=a["stddev"], tab_ptr=z, tab=np.zeros(0), brk_ptr=z,
            brk=np.zeros(0, np.int32), root_id=self.root, scope=list(range(self.F)), feature_type=self.feature_type,
            name=self.name, query={"batch_size": batch_size, "error_kind": error_kind, "max_error": max_error,
                                   "support_marginal": support_marginal})


def config5(seed=1005, num_features=784, depth=4, repetitions=16, width=32, mean_dist=(0.5, 0.3), sd_range=(0.2, 1.0)):
    """RAT-SPN-style layered SPN: `repetitions` random balanced region trees of depth `depth` over
    `num_features` features; every leaf region carries `width` factorised Gaussian distributions, every
    inner region `width` sum nodes over the width x width cross products of its two child regions (dense
    width x width^2 weights ~ Dirichlet(1)); one root sum mixes the root products of all repetitions.
    The full size (784, 4, 16, 32) has ~660 k nodes and ~7.4 M sum edges.  Leaf means ~ N(mean_dist[0], mean_dist[1]),
    standard deviations ~ U(sd_range[0], sd_range[1])."""
    rng = np.random.default_rng(seed)
    K, F = width, num_features
    kind, scope_id, mean, stddev, cnt, child, weight = [], [], [], [], [], [], []
    next_id = 0

    def add(k, n, counts, children, weights=None, scope=None, mu=None, sd=None):
        nonlocal next_id
        ids = np.arange(next_id, next_id + n, dtype=np.int64)
        next_id += n
        kind.append(np.full(n, k, np.int64))
        scope_id.append(np.zeros(n, np.int64) if scope is None else scope)
        mean.append(np.zeros(n) if mu is None else mu)
        stddev.append(np.ones(n) if sd is None else sd)
        cnt.append(np.asarray(counts, np.int64))
        if children is not None:
            child.append(np.asarray(children, np.int32).ravel())
            weight.append(np.zeros(child[-1].size) if weights is None else np.asarray(weights, np.float64).ravel())
        return ids

    root_products = []
    for _ in range(repetitions):
        perm = rng.permutation(F)
        regions = [np.sort(part) for part in np.array_split(perm, 2 ** depth)]
        level = []
        for feats in regions:
            nf = len(feats)
            g = add(wire.K_GAUSS, K * nf, np.zeros(K * nf), None, scope=np.tile(feats, K),
                    mu=rng.normal(mean_dist[0], mean_dist[1], K * nf), sd=rng.uniform(sd_range[0], sd_range[1], K * nf))
            level.append(add(wire.K_PRODUCT, K, np.full(K, nf), g.reshape(K, nf)))
        for d in range(depth - 1, -1, -1):
            nxt = []
            for a_ids, b_ids in zip(level[0::2], level[1::2]):
                pairs = np.stack([np.repeat(a_ids, len(b_ids)), np.tile(b_ids, len(a_ids))], axis=1)
                prods = add(wire.K_PRODUCT, len(pairs), np.full(len(pairs), 2), pairs)
                if d == 0:
                    root_products.append(prods)
                    nxt.append(prods)
                else:
                    w = rng.dirichlet(np.ones(len(prods)), size=K)
                    w = np.maximum(w, 1e-9)
                    w /= w.sum(axis=1, keepdims=True)
                    nxt.append(add(wire.K_SUM, K, np.full(K, len(prods)), np.tile(prods, K), w))
            level = nxt
    allp = np.concatenate(root_products)
    w = np.maximum(rng.dirichlet(np.ones(len(allp))), 1e-9)
    root = add(wire.K_SUM, 1, [len(allp)], allp, w / w.sum())[0]
    arrays = {"kind": np.concatenate(kind), "scope_id": np.concatenate(scope_id), "mean": np.concatenate(mean),
              "stddev": np.concatenate(stddev), "child_id": np.concatenate(child), "weight": np.concatenate(weight)}
    arrays["child_ptr"] = np.concatenate(([0], np.cumsum(np.concatenate(cnt))))
    return ArraySPN(F, "float32", "cfg5_ratspn", arrays, int(root))


def config5_inputs(n, seed=2005, num_features=784):
    return np.random.default_rng(seed).random((n, num_features), dtype=np.float32)
