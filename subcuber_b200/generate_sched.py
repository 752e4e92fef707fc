"""Schedule generator B: postsum placement, presum selection and postsum fusion for a set partition of the
products, with a global-load cost model.

Public surface and printed output follow the reference project's src/generate_sched.py: `gen_schedule(C, Ms, m, n,
k, tile, regtile)` and the helpers it is built from.  For one level of Strassen-Winograd it decides
  * which MiSet (set of products computed by one kernel) produces each postsum expression v1, v2, v3, c0..c3 and
    which MiSets must load it (`set_def_of_postsum_exprs`),
  * which presums are worth materialising in global memory, at most MAX_PRESUM_BUFFERS of them, most used first
    (`apply_presum`), and who computes them (`set_presum_computation`),
  * which MiSets are fused into one launch and whether a hand-over goes through registers, shared memory or
    global memory (`postsum_fusion`), and the launch order (`order_Mis`),
  * an estimate of global loads per partitioning (`get_gmem_loads`).

Behaviour notes kept from the reference so that results agree (tests/test_frontend.py pins them):
  * only the all-singletons partition is evaluated by default (src/generate_sched.py:685); `partitions="all"`
    lifts that restriction for partitions the cost model can size (parts of 1, 2 or 4 products);
  * when the uses of a common expression are merged, they are merged into the group of the LAST MiSet of the
    partitioning (src/generate_sched.py:485-497), which is what yields the {m2, m3, m6, m4} launch.
Iteration orders that the reference takes from Python sets are taken from list order here.
"""
from __future__ import annotations

import argparse
from functools import reduce
from typing import Dict, Iterable, List, Sequence

from .dsl import BinOp, FusedMiSet, Matrix, MiSet

MAX_LEN_PARTITION = 2
MAX_PRESUM_BUFFERS = 2
MAX_FUSED = 4


def get_all_set_partitions(items: Sequence) -> Iterable[List[list]]:
    """All set partitions of `items` (Bell-number many), smaller problems first."""
    if not items:
        yield []
        return
    head, tail = items[0], items[1:]
    for partial in get_all_set_partitions(tail):
        for i, block in enumerate(partial):
            yield partial[:i] + [block + [head]] + partial[i + 1:]
        yield [[head]] + partial


class Partitioning:
    """One evaluated partition: its MiSets, who defines which postsum expression, the presums to materialise and
    the global-load estimate."""

    def __init__(self, common_exprs, misetnodes, expr_def_by_miset, presums_todo, a_gmem_loads, b_gmem_loads,
                 c_gmem_loads):
        self.common_exprs = common_exprs
        self.misetnodes = misetnodes
        self.expr_def_by_miset = expr_def_by_miset
        self.presums_todo = presums_todo
        self.a_gmem_loads, self.b_gmem_loads, self.c_gmem_loads = a_gmem_loads, b_gmem_loads, c_gmem_loads
        self.fused_mi_sets = None
        self.nodes_wo_presum: list = []

    def init_misetnodes_wo_presum(self, mis_wo_presum):
        self.nodes_wo_presum = [node for node in self.misetnodes
                                if len(node.miset) == 1 and node.miset[0] in mis_wo_presum]
        return self.nodes_wo_presum

    def misetnodes_wo_presum(self):
        return self.nodes_wo_presum

    def total_gmem_loads(self):
        return self.a_gmem_loads + self.b_gmem_loads + self.c_gmem_loads

    def partitioning(self):
        return [list(node.miset) for node in self.misetnodes]

    def set_fused_mi_sets(self, fused):
        self.fused_mi_sets = fused

    def get_fused_miset_for_miset(self, node):
        return next((f for f in self.fused_mi_sets if node in f.misets), node)

    def __repr__(self):
        return (repr(self.partitioning()) + " " + repr(self.total_gmem_loads()) + " "
                + repr([p[0] for p in self.presums_todo["a"]]) + " " + repr([p[0] for p in self.presums_todo["b"]]))

    __str__ = __repr__

    def print_miset_in_order(self, order):
        for node in order:
            print(node.full_str())


def all_miset_of_powerto(partitioning, all_mis_len) -> bool:
    """Parts must hold 1, 2, 4 or all products, and at most MAX_LEN_PARTITION of them."""
    return all(len(part) <= MAX_LEN_PARTITION and len(part) in (1, 2, 4, all_mis_len) for part in partitioning)


def atleast_one_miset_wo_presum_is_not_fused(partitioning, Ms) -> bool:
    return any(len(part) == 1 and part[0] in Ms for part in partitioning)


def find_times_each_expr_is_used(C, Ms):
    """Postsum sub-expressions ordered by how often the outputs reach them (most shared first), followed by the
    four outputs themselves."""
    outputs = C.parts
    uses: Dict[Matrix, int] = {}

    def count(node, *_):
        if isinstance(node, BinOp):
            if node not in outputs and node not in Ms:
                uses[node] = uses.get(node, 0) + 1
            if node.op == "@":
                return False
        return True

    C.visit(count)
    ranked = [expr for expr, _ in sorted(uses.items(), key=lambda kv: kv[1], reverse=True)]
    return ranked + outputs


def misetnodes_has_cycle(misetnodes) -> bool:
    done, path = set(), []

    def walk(node) -> bool:
        if node in path:
            return True
        if node in done:
            return False
        done.add(node)
        path.append(node)
        if any(walk(use[1]) for use in node.uses_stores):
            return True
        path.remove(node)
        return False

    return any(node not in done and walk(node) for node in misetnodes)


def set_def_of_postsum_exprs(Cs, partitioning, misetnodes, common_exprs):
    """Assign every postsum expression to the MiSet that completes it.  For `e = x (+|-) y` with x and y defined by
    different MiSets, the MiSet of y loads x from the MiSet of x and stores e (so sums grow along the order
    m0 -> m2 -> m3 ...).  Expressions whose products need no presum at all (c0) are scheduled first."""
    expr_def = {expr: None for expr in common_exprs}

    def needs_presum(expr) -> bool:
        return any(len(mi.get_base_matrices_op1()) != 1 or len(mi.get_base_matrices_op2()) != 1
                   for mi in expr.get_matmul_matrices())

    no_presum = [expr for expr in common_exprs if not needs_presum(expr)]
    common_exprs = no_presum + [expr for expr in common_exprs if expr not in no_presum]

    for expr in common_exprs:
        for operand in (expr.op1, expr.op2):
            for idx, part in enumerate(partitioning):
                if operand in part:
                    expr_def[operand] = misetnodes[idx]

    for expr in common_exprs:
        first, second = expr_def[expr.op1], expr_def[expr.op2]
        if first == second:
            expr_def[expr] = first
            first.add_store(expr)
            continue
        earlier, later = expr.op1, expr.op2
        if expr in no_presum and len(first.miset) != 1 and len(second.miset) == 1:
            earlier, later = expr.op2, expr.op1
        producer, consumer = expr_def[earlier], expr_def[later]
        producer.add_store(earlier)
        producer.uses_stores.append((earlier, consumer))
        consumer.add_load(earlier, misetnodes.index(producer))
        consumer.add_store(expr)
        expr_def[expr] = consumer
    return expr_def, common_exprs


def apply_presum(misetnodes):
    """Pick the presums to materialise: per operand side the sub-expression used by most MiSets, alternating
    a, b, a, b ... until MAX_PRESUM_BUFFERS are chosen.  Returns {"a": [(expr, [using MiSets])], "b": [...]}"""
    users = {"a": {}, "b": {}}
    for node in reversed(misetnodes):
        for side in ("a", "b"):
            for mi in node.miset:
                operand = mi.op1 if side == "a" else mi.op2
                if isinstance(operand, BinOp):
                    for sub in _children_in_order(operand):
                        if isinstance(sub, BinOp):
                            users[side].setdefault(sub, []).append(node)
    ranked = {side: sorted(users[side].items(), key=lambda kv: len(kv[1]), reverse=True) for side in ("a", "b")}
    todo = {"a": [], "b": []}
    chosen, rank = 0, 0
    while rank < len(ranked["a"]) and chosen < MAX_PRESUM_BUFFERS:
        for side in ("a", "b"):
            if chosen >= MAX_PRESUM_BUFFERS:
                break
            todo[side].append(ranked[side][rank])
            chosen += 1
        rank += 1
    return todo


def _children_in_order(expr: BinOp) -> List[Matrix]:
    """Nodes of the subtree of `expr`, outermost first (a deterministic stand-in for get_all_children)."""
    out, seen, todo = [], set(), [expr]
    while todo:
        node = todo.pop(0)
        if node in seen:
            continue
        seen.add(node)
        out.append(node)
        if isinstance(node, BinOp):
            todo += [node.op1, node.op2]
        elif node.parent is not None:
            todo.append(node.parent)
    return out


def set_presum_computation(partitioning_info, mis_wo_presum):
    """The first MiSet that needs no presum (m0) computes every chosen presum; its users load it from there,
    dropping presum loads that the materialised presum makes redundant."""
    maker = partitioning_info.misetnodes_wo_presum()[0]
    maker_idx = partitioning_info.misetnodes.index(maker)
    for side in ("a", "b"):
        for presum, users in partitioning_info.presums_todo[side]:
            maker.presum_stores[side].append(presum)
            if len(users) <= 1:
                for node in users:
                    node.presum_loads[side].append((presum, maker_idx))
                continue
            inside = presum.get_all_children()
            for node in users:
                if node is maker:
                    continue
                keep = []
                for load in node.presum_loads[side]:
                    redundant = load[0] in inside and all(
                        isinstance(op, BinOp) and presum in op.get_all_children()
                        for op in ((mi.op1 if side == "a" else mi.op2) for mi in node.miset))
                    if not redundant:
                        keep.append(load)
                node.presum_loads[side] = keep + [(presum, maker_idx)]


def order_Mis(Cs, partitioning):
    """Launch order of the fused sets: walk the postsum expressions in scheduling order and emit producers before
    consumers."""
    order = []
    nodes = partitioning.misetnodes
    for expr in partitioning.common_exprs:
        chain = []
        for candidate in (partitioning.expr_def_by_miset[expr.op1], partitioning.expr_def_by_miset[expr.op2],
                          partitioning.expr_def_by_miset[expr]):
            if candidate not in chain:
                chain.append(candidate)
        if len(chain) > 1:
            second_reads_first = any(nodes[load.index] == chain[0] for load in chain[1].loads)
            chain = chain if second_reads_first else [chain[1], chain[0]]
        for node in chain:
            fused = partitioning.get_fused_miset_for_miset(node)
            if fused not in order:
                order.append(fused)
    return order


def postsum_fusion(partitioning_info, sorted_common_exprs_and_uses):
    """Fuse MiSets into launches and place every postsum hand-over.

    Fusion: for each common expression (most shared first) walk back from its producer along the postsum loads and
    merge a loaded MiSet into the loader's group when the group stays within MAX_FUSED, both hold equally many
    products and the loaded one is not a no-presum MiSet; then merge the users of the expression (see module
    docstring for the group they join).  Placement inside a fused set: the value produced right before its use in
    the topological order goes through registers ("reg"); one shared-memory buffer ("sh_0") carries the first
    value that lives across more than one step; everything else goes through global memory ("gl").
    """
    slots = {"Registers": 1, "SharedMemory": 1}
    nodes = partitioning_info.misetnodes
    if len(nodes) == 1:
        return
    group = {node: [node] for node in nodes}  # node -> shared list object of its group

    def merge(into, other):
        target = group[into]
        for member in list(group[other]):
            if member not in target:
                target.append(member)
            group[member] = target

    no_presum_nodes = partitioning_info.misetnodes_wo_presum()
    for expr in sorted_common_exprs_and_uses:
        producer = next((node for node in nodes if node.get_store(expr) is not None), None)
        todo = [producer] if producer is not None else []
        while todo:
            parent = todo.pop(0)
            for load in parent.loads:
                child = nodes[load.index]
                if (len(group[parent]) + len(group[child]) <= MAX_FUSED and len(parent.miset) == len(child.miset)
                        and child not in no_presum_nodes):
                    merge(parent, child)
                todo.append(child)
        anchor = nodes[-1]
        for user in [node for node in nodes if node.get_load(expr) is not None]:
            if len(group[anchor]) + len(group[user]) <= MAX_FUSED and len(anchor.miset) == len(user.miset):
                merge(anchor, user)

    fused_lists = []
    for node in nodes:
        if not any(group[node] is seen for seen in fused_lists):
            fused_lists.append(group[node])
    fused_sets = [FusedMiSet(nodes, [n for n in nodes if n in members]) for members in fused_lists]
    partitioning_info.set_fused_mi_sets(fused_sets)

    for fused in fused_sets:
        order = fused.dfs_topo_order()
        if slots["Registers"] > 0:
            for producer, consumer in zip(order, order[1:]):
                for load in consumer.loads:
                    store = producer.get_store(load.expr)
                    if store is not None:
                        store.mem_types.append("reg")
                        load.mem_types.append("reg")
        if slots["SharedMemory"] > 0:
            buffers = [{"buff": b, "status": "avail"} for b in range(slots["SharedMemory"])]
            for store, (start, end) in fused.live_ranges(order):
                for buf in buffers:
                    if buf["status"] != "avail" and buf["status"][1] > end:
                        buf["status"] = "avail"
                for buf in buffers:
                    if buf["status"] == "avail" and end > start + 1:
                        buf["status"] = (start, end)
                        label = f"sh_{buf['buff']}"
                        store.mem_types.append(label)
                        for node in order[start:end + 1]:
                            for load in node.loads:
                                if load.expr == store.expr:
                                    load.mem_types.append(label)
                        break

    for node in nodes:
        for load in node.loads:
            if not load.mem_types:
                load.mem_types.append("gl")
                nodes[load.index].get_store(load.expr).mem_types.append("gl")


def get_gmem_loads(misetnodes, presums_todo, Mis, M, N, K, tm, tn, rm, rn):
    """Estimated global loads (elements) of A, B and C for a partitioning with tile (tm, tn) and register tile
    (rm, rn): presum materialisation reads each base quadrant once; every MiSet then loads, per output tile and
    k, one tile row/column per operand it reads (a materialised presum counts as one operand)."""
    a_loads = b_loads = c_loads = 0
    for side in ("a", "b"):
        if presums_todo[side]:
            bases = reduce(lambda x, y: x | y, [entry[0].get_base_matrices() for entry in presums_todo[side]])
            if side == "a":
                a_loads += len(bases) * (M // 2) * (K // 2)
            else:
                b_loads += len(bases) * (N // 2) * (K // 2)

    for node in misetnodes:
        via_presum = {"a": set(), "b": set()}
        direct = {"a": set(), "b": set()}
        for mi in node.miset:
            for side in ("a", "b"):
                todo = [mi.op1 if side == "a" else mi.op2]
                while todo:
                    want = todo.pop(0)
                    if any(want == entry[0] for entry in presums_todo[side]):
                        via_presum[side].add(want)
                    elif isinstance(want, BinOp):
                        todo += [want.op1, want.op2]
                    elif isinstance(want, Matrix):
                        direct[side].add(want)
        m_tiles = (M // tm) // 2 * (N // tn) // 2
        rm_fac, rn_fac = {1: (1, 1), 2: (2, 1), 4: (2, 2)}.get(len(node.miset), (1, 1))
        if len(node.miset) == len(Mis):
            rm_fac = rn_fac = 1
        per_k = rm_fac * rn_fac * m_tiles * (K // 2)
        a_loads += per_k * ((len(via_presum["a"]) + len(direct["a"])) * tm // rm_fac)
        # the B term counts the A-side presums, exactly as the reference's cost model does (src/generate_sched.py:671)
        b_loads += per_k * ((len(via_presum["a"]) + len(direct["b"])) * tn // rn_fac)
    return a_loads, b_loads, c_loads


def gen_schedule(C, Ms, m, n, k, tile, regtile, partitions: str = "singletons"):
    """Evaluate partitions of the products, print the best five with their launches in order
    (reference: src/generate_sched.py:676-711).  Returns the sorted list of Partitioning objects."""
    ranked_exprs = find_times_each_expr_is_used(C, Ms)
    mis_wo_presum = {Ms[0], Ms[1]}
    valid, considered = [], 0
    for partitioning in get_all_set_partitions(list(Ms)):
        if partitions == "singletons" and any(len(part) != 1 for part in partitioning):
            continue
        if partitions == "singletons":
            partitioning = [[mi] for mi in Ms]
        considered += 1
        if not all_miset_of_powerto(partitioning, len(Ms)):
            continue
        if MAX_PRESUM_BUFFERS > 0 and not atleast_one_miset_wo_presum_is_not_fused(partitioning, mis_wo_presum):
            continue
        nodes = [MiSet(part) for part in partitioning]
        expr_def, common_exprs = set_def_of_postsum_exprs(C.parts, partitioning, nodes, list(ranked_exprs))
        if misetnodes_has_cycle(nodes):
            continue
        presums_todo = apply_presum(nodes)
        a_loads, b_loads, c_loads = get_gmem_loads(nodes, presums_todo, Ms, m, n, k, tile[0], tile[1], regtile[0],
                                                   regtile[1])
        valid.append(Partitioning(common_exprs, nodes, expr_def, presums_todo, a_loads, b_loads, c_loads))

    print(f"Valid {len(valid)} partitionings out of total {considered}")
    ranked = sorted(valid, key=lambda p: p.total_gmem_loads())
    for p in ranked[:5]:
        p.init_misetnodes_wo_presum(mis_wo_presum)
        set_presum_computation(p, mis_wo_presum)
        postsum_fusion(p, ranked_exprs)
        order = order_Mis(C.parts, p)
        print(p)
        p.print_miset_in_order(order)
        print("\n")
    return ranked


def parse_args(argv=None):
    parser = argparse.ArgumentParser(description="Generate schedule for Strassen variants")
    parser.add_argument("--m", type=int, default=1024, help="Rows of matrix A/C")
    parser.add_argument("--n", type=int, default=1024, help="Columns of matrix B/C")
    parser.add_argument("--k", type=int, default=1024, help="Columns of matrix A / rows of matrix B")
    parser.add_argument("--algo", type=str, default="strassen_winograd", help="Algorithm name")
    parser.add_argument("--level", type=int, default=1, help="Recursion level")
    parser.add_argument("--datatype", type=str, default="fp32", help="Datatype (for metadata/planning)")
    parser.add_argument("--output_dir", type=str, default=".", help="Output directory for generated artifacts")
    return parser.parse_args(argv)


def build(m, n, k, algo, level, datatype, output_dir):
    """Print the level-1 schedule analysis and emit the artefacts of `compile.build` for the Blackwell target."""
    if algo != "strassen_winograd":
        raise ValueError(f"Unsupported algo '{algo}'. Supported: strassen_winograd")
    if level > 2:
        raise ValueError(f"Unsupported level '{level}'. Current implementation supports level <= 2")
    from . import compile as _compile
    from .algos.strassen_winograd_level1 import strassen_winograd

    c, mis = strassen_winograd(m, n, k)
    gen_schedule(c, mis, m, n, k, (128, 256, 64), (8, 8))
    return _compile.build(level, m, n, k, datatype, output_dir, hw="B200")


if __name__ == "__main__":
    args = parse_args()
    build(args.m, args.n, args.k, args.algo, args.level, args.datatype, args.output_dir)
