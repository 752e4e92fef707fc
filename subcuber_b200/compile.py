"""Schedule generator A: which kernels run the products of a (recursive) Strassen-Winograd GEMM, and which of
them are fused into one launch.

Public surface and results follow the reference project's src/compile.py: `HW_SPECS`, `StrassenCompiler`
(`gen_sched`, `iter_all_schedules`, `count_all_schedules`, `output_sum_fusion`, `should_use_k2`, ...) and
`build(level, m, n, k, datatype, output_dir, dry_run, hw, print_all_recursive, print_all_schedules)`.
Kernel vocabulary of the schedules (reference: src/compile.py:206-212,511-531):
    K2(x)  all seven products of x inside one tile kernel
    K1(x)  the product that needs no presum, which also produces the presums
    K4(x)  one product reading presums

Two things differ on purpose:
  * `HW_SPECS` has a "B200" entry, and `build(..., hw="B200")` maps the schedule onto the Blackwell kernels of
    this library (`emit.plan_for_schedule`) and writes real artefacts (schedule, tile programs as JSON and as a C
    table) instead of copying example sources.  The reference's emitter is a file copy from paths that no
    longer exist (src/compile.py:48-131); here nothing is copied.
  * Iteration orders that the reference leaves to Python set ordering are made deterministic.
"""
from __future__ import annotations

import argparse
import collections
import json
import math
import os
from typing import Dict, Iterator, List, Optional

# reference: src/compile.py:8-11, plus the part this library targets
HW_SPECS = {
    "A100": {"sm_count": 108, "shared_mem_per_sm": 168 * 1024, "regs_per_thread": 255},
    "H200": {"sm_count": 132, "shared_mem_per_sm": 228 * 1024, "regs_per_thread": 255},
    "B200": {"sm_count": 148, "shared_mem_per_sm": 227 * 1024, "regs_per_thread": 255, "tmem_columns": 512,
             "l2_bytes": 126 * 1024 * 1024},
}


def _label_token(label: str) -> str:
    lo, hi = label.find("("), label.rfind(")")
    return label if lo < 0 or hi <= lo else label[lo + 1:hi]


class StrassenCompiler:
    # tile sizes the cost heuristics assume (reference: src/compile.py:134-143)
    KernelInfoFP32 = {
        "K2": {"DataType": "fp32", "TileSize": (128, 128), "SharedMemoryBytes": 64 * 1024},
        "K1": {"DataType": "fp32", "TileSize": (256, 128), "SharedMemoryBytes": 64 * 1024},
        "K4": {"DataType": "fp32", "TileSize": (256, 128), "SharedMemoryBytes": 64 * 1024},
    }
    KernelInfoFP16 = {
        "K2": {"DataType": "fp32", "TileSize": (128, 128), "SharedMemoryBytes": 64 * 1024},
        "K1": {"DataType": "fp32", "TileSize": (256, 128), "SharedMemoryBytes": 96 * 1024},
        "K4": {"DataType": "fp32", "TileSize": (256, 128), "SharedMemoryBytes": 96 * 1024},
    }

    def __init__(self, hw_name: str = "A100", print_all_recursive: bool = False):
        self.hw = HW_SPECS.get(hw_name)
        self.hw_name = hw_name
        self.memo: Dict = {}
        self.fusion_memo: Dict = {}
        self.last_fusion_schedule = None
        self.print_all_recursive = print_all_recursive

    # ------------------------------------------------------------------------------------------ helpers
    def _trace_schedule(self, level, mnk, src_m, schedule, from_memo=False):
        if self.print_all_recursive:
            tag = " [memo]" if from_memo else ""
            print(f"[Trace] level={level}, mnk={mnk}, src={src_m if src_m is not None else 'Base'}{tag} -> {schedule}")

    def build_output_sum_dag(self, root_node):
        """(dag, products): the products of the algorithm in discovery order (operands before users, left before
        right).  Like the reference (src/compile.py:166-190) the dependency dict is returned empty: fusion falls
        back to the discovery chain."""
        found = []

        def collect(node, *_):
            if getattr(node, "op", None) == "@":
                found.append(node)
                return False
            return True

        if hasattr(root_node, "visit"):
            root_node.visit(collect)
        return collections.defaultdict(list), list(dict.fromkeys(found))

    def get_min_input_sum_loads(self, sub_matmuls):
        """The product that needs no extra quadrant loads for presums: m0 = a0 b0 for Strassen-Winograd."""
        return sub_matmuls[0]

    def estimate_cost(self, schedule, mnk):
        m, n, k = mnk
        return m * n * k * (0.8 if ("K2" in str(schedule) and m < 2048) else 1.0)

    def should_use_k2(self, mnk) -> bool:
        """All-in-one tile kernel strictly below 2048 in every dimension (reference: src/compile.py:206-212)."""
        return all(d < 2048 for d in mnk)

    def count_all_schedules(self, level: int) -> int:
        if level <= 0:
            return 0
        return 2 if level == 1 else self.count_all_schedules(level - 1) ** 6

    # ------------------------------------------------------------------------------------- enumeration
    def iter_all_schedules(self, alg_func, level, mnk, src_m=None) -> Iterator[list]:
        """Every schedule of `level` levels: 2 at level 1, and for deeper levels every combination of child
        schedules under the six K4 branches (reference: src/compile.py:222-257)."""
        root, products = alg_func(*mnk)
        _, order = self.build_output_sum_dag(root)
        first = self.get_min_input_sum_loads(products)
        rest = [p for p in order if p != first]
        if level == 1:
            yield [f"K2({src_m if src_m else 'Base'})"]
            yield [f"K1({first})"] + [f"K4({p})" for p in rest]
            return
        half = (mnk[0] // 2, mnk[1] // 2, mnk[2] // 2)

        def expand(i: int, chosen: list):
            if i == len(rest):
                yield list(chosen)
                return
            for child in self.iter_all_schedules(alg_func, level - 1, half, rest[i]):
                chosen.append({f"K4({rest[i]})": child})
                yield from expand(i + 1, chosen)
                chosen.pop()

        for combo in expand(0, []):
            yield [f"K1({first})"] + combo

    # ------------------------------------------------------------------------------------------ fusion
    def output_sum_fusion(self, dag, schedule, mnk, kernel_type):
        """Greedy fusion of K2 or K4 launches along the output-sum chain (reference: src/compile.py:259-478).

        A parent and a user are merged when: neither is a K1; the parent's group has fewer than 2 fused uses
        (two hand-over buffers); the merged group has at most 4 kernels; the merge creates no cycle between
        groups; and enough thread blocks remain to fill the SMs (groups_after * blocks_per_kernel > sm_count).
        """
        if kernel_type not in ("K2", "K4"):
            return {"kernel": kernel_type, "fused_map": {}, "groups": [], "notes": "Unsupported kernel type for fusion"}
        prefix = kernel_type + "("
        targets = []
        for item in schedule:
            if isinstance(item, str):
                if item.startswith(prefix):
                    targets.append(item)
            elif isinstance(item, dict):
                targets.extend(key for key in item if key.startswith(prefix))
        if not targets:
            return {"kernel": kernel_type, "fused_map": {}, "groups": [],
                    "notes": f"No {kernel_type} kernels available for fusion"}

        # edges between scheduled kernels, projected from the expression DAG; chain fallback when it has none
        by_token = {_label_token(t): t for t in targets}
        edges = {t: [] for t in targets}
        projected = 0
        for parent, users in dag.items():
            src = next((lab for tok, lab in by_token.items() if tok in str(parent)), None)
            if src is None:
                continue
            for user in users:
                dst = next((lab for tok, lab in by_token.items() if tok in str(user)), None)
                if dst is not None and dst != src and dst not in edges[src]:
                    edges[src].append(dst)
                    projected += 1
        if projected == 0:
            for a, b in zip(targets, targets[1:]):
                edges[a].append(b)

        def topo(adj):
            indeg = {n: 0 for n in adj}
            for kids in adj.values():
                for kid in kids:
                    if kid in indeg:
                        indeg[kid] += 1
            ready = collections.deque(n for n, d in indeg.items() if d == 0)
            out, seen = [], set()
            while ready:
                n = ready.popleft()
                if n in seen:
                    continue
                seen.add(n)
                out.append(n)
                for kid in adj.get(n, []):
                    if kid in indeg:
                        indeg[kid] -= 1
                        if indeg[kid] == 0:
                            ready.append(kid)
            return out + [n for n in adj if n not in seen]

        def reaches(adj, src, dst):
            if src == dst:
                return True
            seen, todo = {src}, collections.deque([src])
            while todo:
                for nxt in adj.get(todo.popleft(), []):
                    if nxt == dst:
                        return True
                    if nxt not in seen:
                        seen.add(nxt)
                        todo.append(nxt)
            return False

        def group_graph(groups):
            g = {tuple(sorted(members)): set() for members in groups.values()}
            for parent, kids in edges.items():
                pr = tuple(sorted(groups[parent]))
                for kid in kids:
                    kr = tuple(sorted(groups[kid]))
                    if kr != pr:
                        g[pr].add(kr)
            return {k: list(v) for k, v in g.items()}

        tile_m, tile_n = self.KernelInfoFP32[kernel_type]["TileSize"]
        pm, pn = (max(1, mnk[0] // 2), max(1, mnk[1] // 2)) if kernel_type == "K4" else (mnk[0], mnk[1])
        blocks_per_kernel = math.ceil(pm / tile_m) * math.ceil(pn / tile_n)
        sm_count = self.hw["sm_count"] if self.hw else 1
        max_fused, hand_over_buffers = 4, 2

        groups = {t: {t} for t in targets}
        progress = True
        while progress:
            progress = False
            for parent in topo(edges):
                pg = groups[parent]
                for user in [u for u in edges.get(parent, []) if groups[u] is not pg]:
                    ug = groups[user]
                    if parent.startswith("K1(") or user.startswith("K1("):
                        continue
                    fused_uses = {u for p in pg for u in edges.get(p, []) if groups[u] is pg}
                    if len(fused_uses) >= hand_over_buffers:
                        continue
                    merged = pg | ug
                    if len(merged) > max_fused:
                        continue
                    if reaches(group_graph(groups), tuple(sorted(ug)), tuple(sorted(pg))):
                        continue
                    remaining = max(1, len({tuple(sorted(g)) for g in groups.values()}) - 1)
                    if remaining * blocks_per_kernel <= sm_count:
                        continue
                    for node in merged:
                        groups[node] = merged
                    pg = merged
                    progress = True

        unique = []
        for members in groups.values():
            ordered = sorted(members)
            if ordered not in unique:
                unique.append(ordered)
        return {
            "kernel": kernel_type,
            "fused_map": {node: sorted(members) for node, members in groups.items()},
            "groups": unique,
            "mnk": mnk,
            "sm_count": sm_count,
            "tb_per_kernel": blocks_per_kernel,
            "dag_edges": sum(len(v) for v in edges.values()),
        }

    # -------------------------------------------------------------------------------------- selection
    def gen_sched(self, alg_func, level, mnk, src_m=None):
        """Pick the schedule for `level` levels on an mnk problem (reference: src/compile.py:480-560).

        Level 1: K2 when every dimension is below 2048, else K1 + six K4.  Deeper levels: K1 for the first
        product and the (memoised) schedule of the half-size problem under each K4 branch.  Results are memoised
        per (level, mnk), so, as in the reference, the label inside a memoised child schedule is the one of the
        first branch that computed it.
        """
        key = (level, mnk)
        if key in self.memo:
            self.last_fusion_schedule = self.fusion_memo.get(key)
            self._trace_schedule(level, mnk, src_m, self.memo[key], from_memo=True)
            return self.memo[key]
        root, products = alg_func(*mnk)
        dag, order = self.build_output_sum_dag(root)
        first = self.get_min_input_sum_loads(products)
        rest = [p for p in order if p != first]

        if level == 1:
            if self.should_use_k2(mnk):
                schedule = [f"K2({src_m if src_m else 'Base'})"]
                fusion = self.output_sum_fusion(dag, schedule, mnk, kernel_type="K2")
            else:
                schedule = [f"K1({first})"] + [f"K4({p})" for p in rest]
                fusion = self.output_sum_fusion(dag, schedule, mnk, kernel_type="K4")
        else:
            def count_k2(node) -> int:
                if isinstance(node, str):
                    return 1 if node.startswith("K2(") else 0
                if isinstance(node, list):
                    return sum(count_k2(x) for x in node)
                if isinstance(node, dict):
                    return sum((1 if isinstance(k, str) and k.startswith("K2(") else 0) + count_k2(v)
                               for k, v in node.items())
                return 0

            half = (mnk[0] // 2, mnk[1] // 2, mnk[2] // 2)
            schedule = [f"K1({first})"]
            many_k2 = False
            for p in rest:
                child = self.gen_sched(alg_func, level - 1, half, p)
                many_k2 = many_k2 or count_k2(child) > 1
                schedule.append({f"K4({p})": child})
            fusion = self.output_sum_fusion(dag, schedule, mnk, kernel_type="K2" if many_k2 else "K4")

        self.memo[key] = schedule
        self.fusion_memo[key] = fusion
        self.last_fusion_schedule = fusion
        self._trace_schedule(level, mnk, src_m, schedule)
        return schedule


def build(level, m, n, k, datatype, output_dir, dry_run=False, hw="A100", print_all_recursive=False,
          print_all_schedules=False, algorithm="strassen_winograd"):
    """Generate the schedule and emit the artefacts for it.  Signature of the reference's `build`
    (src/compile.py:563-653) plus `algorithm` ("strassen_winograd", or "strassen" for Strassen's original algorithm,
    level 1); returns the final schedule, or the list of all schedules when `print_all_schedules` is set (which
    implies a dry run).

    Artefacts written to `output_dir` (or listed, with `dry_run`): `schedule.json` (schedule, fusion groups and
    the Blackwell launch plan) and, for level 1, `tile_programs.json` / `sw_tile_programs.inc`: the per-tile
    programs of each launch in the form the CUDA kernels interpret.
    """
    from . import emit
    from .algos.strassen_level1 import strassen
    from .algos.strassen_winograd_level1 import strassen_winograd

    if algorithm not in ("strassen_winograd", "strassen"):
        raise ValueError(f"Unsupported algorithm '{algorithm}'. Supported: strassen_winograd, strassen")
    alg_func = strassen_winograd if algorithm == "strassen_winograd" else strassen
    dtype = datatype.lower()
    if dtype not in ("fp32", "f32", "fp16", "f16"):
        raise ValueError(f"Unsupported datatype '{datatype}'. Supported: f32, f16")
    effective_dry_run = dry_run or print_all_schedules
    compiler = StrassenCompiler(hw_name=hw, print_all_recursive=print_all_recursive)

    if print_all_schedules:
        total = compiler.count_all_schedules(level)
        print(f"Total schedules at level {level}: {total}")
        found = []
        try:
            for idx, schedule in enumerate(compiler.iter_all_schedules(alg_func, level=level, mnk=(m, n, k)), 1):
                print(f"Schedule {idx}/{total}: {schedule}")
                kernel = "K2" if "K2(" in str(schedule) else "K4"
                print(f"Fusion Schedule {idx}/{total}: "
                      f"{compiler.output_sum_fusion(dag={}, schedule=schedule, mnk=(m, n, k), kernel_type=kernel)}")
                found.append(schedule)
        except BrokenPipeError:
            pass
        return found

    final_schedule = compiler.gen_sched(alg_func, level=level, mnk=(m, n, k))
    print(f"Generated Optimal Schedule:\n{final_schedule}")
    print(f"Generated Fusion Schedule:\n{compiler.last_fusion_schedule}")

    plan = emit.plan_for_schedule(final_schedule, level, (m, n, k), "f16" if "16" in dtype else "f32", algorithm)
    files = emit.artefacts(final_schedule, compiler.last_fusion_schedule, plan)
    for name, text in files.items():
        path = os.path.join(output_dir, name)
        if effective_dry_run:
            print(f"[dry-run] would write {path} ({len(text)} bytes)")
        else:
            os.makedirs(output_dir, exist_ok=True)
            with open(path, "w", encoding="utf-8") as f:
                f.write(text)
            print(f"wrote {path}")
    return final_schedule


def main(argv=None):
    parser = argparse.ArgumentParser(description="Generate Strassen kernel schedules")
    parser.add_argument("--level", type=int, required=True, help="Strassen recursion level")
    parser.add_argument("--m", type=int, required=True, help="Matrix M dimension")
    parser.add_argument("--n", type=int, required=True, help="Matrix N dimension")
    parser.add_argument("--k", type=int, required=True, help="Matrix K dimension")
    parser.add_argument("--datatype", type=str, required=True, help="fp32 / fp16")
    parser.add_argument("--output_dir", type=str, required=True, help="Output directory for the emitted artefacts")
    parser.add_argument("--dry-run", action="store_true", help="Preview the writes without touching files")
    parser.add_argument("--hw", type=str, default="A100", choices=sorted(HW_SPECS.keys()), help="Target hardware")
    parser.add_argument("--print-all-recursive", action="store_true", help="Print the schedule of every recursive call")
    parser.add_argument("--print-all-schedules", action="store_true", help="Print all schedules of the level")
    args = parser.parse_args(argv)
    build(level=args.level, m=args.m, n=args.n, k=args.k, datatype=args.datatype, output_dir=args.output_dir,
          dry_run=args.dry_run, hw=args.hw, print_all_recursive=args.print_all_recursive,
          print_all_schedules=args.print_all_schedules)


if __name__ == "__main__":
    main()
