"""Expression DSL for Strassen-like algorithms.

Same public surface as the reference project's front end (src/dsl.py there): `Matrix` (a rectangular view into a
parent matrix), `BinOp` (+, -, @ nodes), `Combine4x4` (the 2x2 block result), and the schedule bookkeeping classes
`MiSet`, `MiSetLoadStore`, `FusedMiSet` that `generate_sched` works on.  An algorithm is written as ordinary Python
arithmetic on quadrant views (see algos/strassen_winograd_level1.py); the result is an expression DAG that the
schedule generators and the tile-program emitter walk.

On top of the reference surface this module adds `expand_terms`, the symbolic expansion the Blackwell emitter needs:
the list of (+-1, quadrant) terms of a presum expression in the evaluation order of the expression tree.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple


class Matrix:
    """A view `parent[r0:r1, c0:c1]` (or a root matrix when `parent` is None).

    `start` is kept in the coordinates of the ROOT matrix; `shape` is (rows, cols).
    (reference: src/dsl.py:3-35)
    """

    def __init__(self, shape, start=(0, 0), parent: Optional["Matrix"] = None):
        self.shape = shape
        origin = parent.start if parent is not None else (0, 0)
        self.start = (origin[0] + start[0], origin[1] + start[1])
        self.parent = parent
        self.name = ""
        self.presum_used_by: list = []

    # -- construction ---------------------------------------------------------------------------------
    def __getitem__(self, key) -> "Matrix":
        if len(key) != 2:
            raise AssertionError("a matrix view takes exactly two slices")
        begin, extent = [], []
        for size, sl in zip(self.shape, key):
            lo = 0 if sl.start is None else sl.start
            hi = size if sl.stop is None else sl.stop
            begin.append(lo)
            extent.append(hi - lo)
        return Matrix(extent, start=begin, parent=self)

    def __add__(self, other: "Matrix") -> "BinOp":
        return BinOp(self, other, "+")

    def __sub__(self, other: "Matrix") -> "BinOp":
        return BinOp(self, other, "-")

    def __matmul__(self, other: "Matrix") -> "BinOp":
        return BinOp(self, other, "@")

    # -- naming / printing ----------------------------------------------------------------------------
    def var_names(self, frame_locals: Dict[str, object]) -> None:
        """Give every Matrix found in `frame_locals` (typically `locals()`) the name of its variable."""
        for label, value in frame_locals.items():
            if isinstance(value, Matrix):
                value.name = label

    def __str__(self) -> str:
        return self.name

    __repr__ = __str__

    def visit(self, visitor: Callable, *visitor_args) -> None:
        """Pre-order walk towards the roots; `visitor(node, args)` returns False to prune."""
        if visitor(self, visitor_args) and self.parent is not None:
            self.parent.visit(visitor, visitor_args)

    def print_tree(self, visited: Optional[Set["Matrix"]] = None) -> None:
        """Print one definition per node, operands before their users (reference: src/dsl.py:54-73)."""
        if visited is None:
            visited = set()
        if self in visited:
            return
        visited.add(self)
        if isinstance(self, BinOp):
            self.op1.print_tree(visited)
            self.op2.print_tree(visited)
            print(f"{self.name} = {self.op1.name} {self.op} {self.op2.name}")
        elif isinstance(self, Combine4x4):
            labels = []
            for part in self.parts:
                part.print_tree(visited)
                labels.append(part.name)
            print(f"{self.name} = {labels}")
        elif self.parent is not None:
            r0, c0 = self.start
            print(f"{self.name} = {self.parent.name}[{r0}:{self.shape[0] + r0}, {c0}:{self.shape[1] + c0}]")
        else:
            print(f"{self.name} = Matrix({self.shape[0]}, {self.shape[1]})")

    # -- queries --------------------------------------------------------------------------------------
    def get_base_matrices(self, stopFn: Optional[Callable[["Matrix"], bool]] = None) -> Set["Matrix"]:
        """Quadrant views (children of a root matrix) this expression reads; `stopFn(node)` cuts the walk and
        reports `node` itself (reference: src/dsl.py:75-87)."""
        if stopFn is not None and stopFn(self):
            return {self}
        if isinstance(self, BinOp):
            return self.op1.get_base_matrices(stopFn) | self.op2.get_base_matrices(stopFn)
        if self.parent is None:
            return set()
        if self.parent.parent is None:
            return {self}
        return self.parent.get_base_matrices(stopFn)


class BinOp(Matrix):
    """`op1 <op> op2` with op in {"+", "-", "@"} (reference: src/dsl.py:89-128)."""

    def __init__(self, m1: Matrix, m2: Matrix, op: str):
        super().__init__((m1.shape[0], m2.shape[1]))
        self.op = op
        self.op1 = m1
        self.op2 = m2

    def get_base_matrices_op1(self) -> Set[Matrix]:
        return self.op1.get_base_matrices()

    def get_base_matrices_op2(self) -> Set[Matrix]:
        return self.op2.get_base_matrices()

    def get_matmul_matrices(self) -> Set[Matrix]:
        """The products (@ nodes) a postsum expression is built from."""
        return set(self.get_base_matrices(stopFn=lambda node: node.op == "@"))

    def get_all_children(self) -> Set[Matrix]:
        found: Set[Matrix] = set()

        def collect(node, *_):
            found.add(node)
            return True

        self.visit(collect)
        return found

    def get_children_at_levels(self) -> Dict[int, List[Matrix]]:
        """Nodes grouped by depth below this node (0 = self)."""
        levels: Dict[int, List[Matrix]] = {}
        todo = deque([(self, 0)])
        while todo:
            node, depth = todo.popleft()
            levels.setdefault(depth, []).append(node)
            if isinstance(node, BinOp):
                todo.append((node.op1, depth + 1))
                todo.append((node.op2, depth + 1))
        return levels

    def visit(self, visitor: Callable, *visitor_args) -> None:
        if visitor(self, visitor_args):
            self.op1.visit(visitor, visitor_args)
            self.op2.visit(visitor, visitor_args)


class Combine4x4(Matrix):
    """The result assembled from four quadrant expressions [c0, c1, c2, c3], row-major quadrant order
    (reference: src/dsl.py:130-138)."""

    def __init__(self, parts: Sequence[Matrix]):
        super().__init__((parts[0].shape[0] * 2, parts[0].shape[1] * 2))
        self.parts = parts

    def visit(self, visitor: Callable, *visitor_args) -> None:
        if visitor(self, visitor_args):
            for part in self.parts:
                part.visit(visitor, visitor_args)


# ----------------------------------------------------------------------------------------------------------
# Schedule bookkeeping (reference: src/dsl.py:141-330)


class MiSetLoadStore:
    """One postsum hand-over: `expr` produced by / read from the MiSet with index `index`, through `mem_types`
    (a load has one memory type, a store may have several)."""

    def __init__(self, expr, misetindex):
        self.expr = expr
        self.index = misetindex
        self.mem_types: List[str] = []

    def __repr__(self) -> str:
        return f"({self.expr!r}, {self.index!r}, {self.mem_types!r})"

    __str__ = __repr__


class MiSet:
    """A set of products computed by one kernel, with the postsum values it stores and loads and the presums it
    computes (presum_stores) or reads (presum_loads), keyed "a" / "b"."""

    small_print = False

    def __init__(self, miset):
        self.miset = miset
        self.stores: List[MiSetLoadStore] = []
        self.loads: List[MiSetLoadStore] = []
        self.uses_stores: list = []      # (expr, consuming MiSet)
        self.common_exprs: list = []
        self.presum_stores = {"a": [], "b": []}
        self.presum_loads = {"a": [], "b": []}

    def get_store(self, expr) -> Optional[MiSetLoadStore]:
        return next((s for s in self.stores if s.expr == expr), None)

    def add_store(self, store) -> None:
        if self.get_store(store) is None:
            self.stores.append(MiSetLoadStore(store, 0))

    def get_load(self, load, src=-1) -> Optional[MiSetLoadStore]:
        return next((l for l in self.loads if l.expr == load and (src == -1 or l.index == src)), None)

    def add_load(self, load, src) -> None:
        if self.get_load(load, src) is None:
            self.loads.append(MiSetLoadStore(load, src))

    def add_presum_load(self, aorb: str, expr, source) -> None:
        if all(existing[0] != expr for existing in self.presum_loads[aorb]):
            self.presum_loads[aorb].append((expr, source))

    def __repr__(self) -> str:
        if MiSet.small_print:
            return "{" + repr(self.miset) + "}"
        return ("{" + repr(self.miset) + ", loads: " + repr(self.loads) + ", stores: " + repr(self.stores) + " || loads: "
                + repr(self.presum_loads) + ", stores: " + repr(self.presum_stores) + "}")

    __str__ = __repr__

    def full_str(self, indent: int = 0) -> str:
        pad = " " * indent
        return (repr(self.miset) + "\n" + pad + "post loads: " + repr(self.loads) + pad + "stores: " + repr(self.stores)
                + "\n" + pad + "pre loads: " + repr(self.presum_loads) + pad + "stores: " + repr(self.presum_stores))


class FusedMiSet:
    """MiSets fused into one launch.  Stores and loads are split into those that cross the boundary of the fused
    set (`stores`, `loads`) and those satisfied inside it (`fused_stores`, `fused_loads`)."""

    def __init__(self, misetnodes, misets):
        self.misets = misets
        self.stores, self.loads, self.fused_stores, self.fused_loads = [], [], [], []
        inside = list(misets)
        for node in inside:
            for store in node.stores:
                read_outside = any(other not in inside and any(l.expr == store.expr for l in other.loads)
                                   for other in misetnodes)
                read_inside = any(any(l.expr == store.expr for l in other.loads) for other in inside)
                if read_outside:
                    self.stores.append(store)
                if read_inside:
                    self.fused_stores.append(store)
        for node in inside:
            for load in node.loads:
                if misetnodes[load.index] in inside:
                    self.fused_loads.append(load)
                else:
                    self.loads.append(load)

    def dfs_topo_order(self):
        """Topological order (producers first) that visits MiSets with several stores first, so that a value
        produced right before its use can stay in registers."""
        seen, post = set(), []

        def descend(node):
            seen.add(node)
            single = [u for u in node.uses_stores if len(u[1].stores) == 1]
            multi = [u for u in node.uses_stores if len(u[1].stores) != 1]
            for use in multi + single:
                if use[1] not in seen and use[1] in self.misets:
                    descend(use[1])
            post.append(node)

        single = [m for m in self.misets if len(m.stores) == 1]
        multi = [m for m in self.misets if len(m.stores) != 1]
        for node in multi + single:
            if node not in seen:
                descend(node)
        return post[::-1]

    def live_ranges(self, linear_order):
        """[(store, [def position, last use position])] for the stores consumed inside the fused set, sorted by
        definition position."""
        spans = {store: [-1, -1] for store in self.fused_stores}
        for store in self.fused_stores:
            for pos, node in enumerate(linear_order):
                if any(store == own for own in node.stores):
                    spans[store][0] = pos
                for load in node.loads:
                    if load.expr == store.expr and load in self.fused_loads:
                        spans[store][1] = pos
        return sorted(spans.items(), key=lambda item: item[1][0])

    def __repr__(self) -> str:
        MiSet.small_print = True
        try:
            return "F" + repr(self.misets)
        finally:
            MiSet.small_print = False

    def full_str(self) -> str:
        return "{\n" + "\n".join(node.full_str(2) for node in self.dfs_topo_order()) + "\n}"


# ----------------------------------------------------------------------------------------------------------
# Addition for the Blackwell emitter


def expand_terms(expr: Matrix) -> List[Tuple[int, Matrix]]:
    """Flatten a presum expression (only + and - over quadrant views) into signed quadrant terms, in an order
    whose left-to-right evaluation reproduces the floating-point result of the expression tree.

    `x - y` with y a sum is expanded as (-y) + x, which is exact because negation is exact and rounding is
    symmetric; e.g. a1 - ((a2 + a3) - a0) becomes [-a2, -a3, +a0, +a1].
    """
    if not isinstance(expr, BinOp):
        return [(1, expr)]
    if expr.op == "@":
        raise ValueError("expand_terms takes presum expressions, not products")
    left, right = expand_terms(expr.op1), expand_terms(expr.op2)
    sign = 1 if expr.op == "+" else -1
    right = [(sign * c, m) for c, m in right]
    if len(right) == 1:
        return left + right
    if len(left) == 1:
        # leaf (+|-) tree: evaluate the tree first, then bring in the leaf
        return right + left
    raise ValueError("sum of two non-trivial subtrees has no single left-to-right order")
