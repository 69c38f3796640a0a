"""Minimal SPN node classes with the attribute names SPFlow uses, so that models can be built
and serialised without SPFlow installed.  Real SPFlow nodes are accepted wherever these are:
the serialiser only looks at the class *name* and at the attributes listed here
(the reference's serialiser touches exactly these: BinarySerialization.py:160-242).

  Sum(weights, children)              .weights .children .scope .id
  Product(children)                   .children .scope .id
  Gaussian(mean, stdev, scope)        .mean .stdev .scope
  Categorical(p, scope)               .p .scope
  Histogram(breaks, densities, bin_repr_points, scope, type_, meta_type)
"""


class Node:
    def __init__(self):
        self.id = 0
        self.scope = []

    @property
    def name(self):
        return "%sNode_%s" % (self.__class__.__name__, self.id)


class Sum(Node):
    def __init__(self, weights=None, children=None):
        Node.__init__(self)
        self.weights = [] if weights is None else weights
        self.children = [] if children is None else children


class Product(Node):
    def __init__(self, children=None):
        Node.__init__(self)
        self.children = [] if children is None else children


class Leaf(Node):
    def __init__(self, scope=None):
        Node.__init__(self)
        if scope is not None:
            self.scope = [scope] if isinstance(scope, int) else list(scope)


class Gaussian(Leaf):
    def __init__(self, mean=None, stdev=None, scope=None):
        Leaf.__init__(self, scope)
        self.mean = mean
        self.stdev = stdev


class Categorical(Leaf):
    def __init__(self, p=None, scope=None):
        Leaf.__init__(self, scope)
        self.p = p


class Histogram(Leaf):
    def __init__(self, breaks, densities, bin_repr_points=None, scope=None, type_=None, meta_type=None):
        Leaf.__init__(self, scope)
        self.breaks = breaks
        self.densities = densities
        self.bin_repr_points = [] if bin_repr_points is None else bin_repr_points
        self.type = type_
        self.meta_type = meta_type


def kind_of(node):
    """'sum' | 'product' | 'gaussian' | 'categorical' | 'histogram' for our nodes and SPFlow's."""
    n = type(node).__name__
    for cls in type(node).__mro__:
        k = {"Sum": "sum", "Product": "product", "Gaussian": "gaussian", "Categorical": "categorical",
             "Histogram": "histogram"}.get(cls.__name__)
        if k:
            return k
    raise NotImplementedError("No serialization defined for node %r of type %s" % (node, n))


def topological_order(root):
    """All nodes reachable from root, children before parents, each once (iterative DFS)."""
    order, seen, stack = [], set(), [(root, 0)]
    while stack:
        node, i = stack.pop()
        ch = getattr(node, "children", None) or []
        if i == 0:
            if id(node) in seen:
                continue
            seen.add(id(node))
        if i < len(ch):
            stack.append((node, i + 1))
            if id(ch[i]) not in seen:
                stack.append((ch[i], 0))
        else:
            order.append(node)
    return order


def assign_ids(root, taken=None):
    """Give every node a file-unique integer id (children first)."""
    taken = {} if taken is None else taken
    for n in topological_order(root):
        n.id = len(taken)
        taken[n.id] = n
    return root


def rebuild_scopes_bottom_up(root):
    for n in topological_order(root):
        ch = getattr(n, "children", None)
        if ch:
            s = set()
            for c in ch:
                s.update(c.scope)
            n.scope = sorted(s)
    return root


def is_valid(root, tol=1e-6):
    """Structural validity: complete sums, decomposable products, normalised weights."""
    for n in topological_order(root):
        k = kind_of(n)
        if k == "sum":
            if len(n.children) == 0 or len(n.children) != len(n.weights):
                return False, "sum %s: children/weights mismatch" % n.id
            if abs(float(sum(n.weights)) - 1.0) > tol:
                return False, "sum %s: weights do not sum to 1" % n.id
            s0 = set(n.children[0].scope)
            if any(set(c.scope) != s0 for c in n.children):
                return False, "sum %s is not complete" % n.id
        elif k == "product":
            if len(n.children) == 0:
                return False, "product %s has no children" % n.id
            tot = sum(len(c.scope) for c in n.children)
            if tot != len(set().union(*[set(c.scope) for c in n.children])):
                return False, "product %s is not decomposable" % n.id
        elif len(n.scope) != 1:
            return False, "leaf %s is not univariate" % n.id
    return True, None
