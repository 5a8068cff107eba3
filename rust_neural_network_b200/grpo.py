"""Group-relative policy optimisation and its companions (rust-nn src/grpo.rs): `GrpoConfig`,
`GrpoGroup`, `GrpoTrainer`, `GrpoStats`; the heuristic multi-dimensional `RewardModel`
(`RewardDimension`, `RewardScore`, `RewardWeights`); the adversarial `CoEvolutionTrainer`
(`ModelRole`, `AdversarialEpisode`, `CoEvolutionStats`); and the repository graph (`FileNode`,
`StructureEdge`, `StructureEdgeType`, `RepoGraph`, `parse_rust_file`).

The reference's `GrpoTrainer.step` only records statistics (src/grpo.rs:104-153). `grpo_loss` adds
the objective those statistics belong to - the clipped surrogate with group-normalised advantages
and a KL penalty against a reference policy - as a tensor function, so a policy built from this
package's modules can actually be trained with it.
"""
from __future__ import annotations

import dataclasses
import enum
import math
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch


@dataclasses.dataclass
class GrpoConfig:
    group_size: int = 8
    clip_eps: float = 0.2
    lr: float = 1e-3
    kl_coeff: float = 0.04
    num_iterations: int = 1


@dataclasses.dataclass
class GrpoGroup:
    prompt: str
    responses: List[str]
    rewards: List[float]

    def advantages(self) -> List[float]:
        n = len(self.rewards)
        if n == 0:
            return []
        mean = sum(self.rewards) / n
        std = max(math.sqrt(sum((r - mean) ** 2 for r in self.rewards) / n), 1e-8)
        return [(r - mean) / std for r in self.rewards]

    def best_index(self) -> int:
        best, bi = -math.inf, 0
        for i, r in enumerate(self.rewards):
            if r >= best:          # the last maximum wins, as Iterator::max_by does
                best, bi = r, i
        return bi

    def best_response(self) -> str:
        return self.responses[self.best_index()]


@dataclasses.dataclass
class GrpoStats:
    step: int
    mean_reward: float
    std_reward: float
    mean_advantage: float
    best_reward: float
    worst_reward: float


def grpo_loss(logp: torch.Tensor, old_logp: torch.Tensor, advantages: torch.Tensor,
              ref_logp: Optional[torch.Tensor] = None, clip_eps: float = 0.2, kl_coeff: float = 0.04,
              mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Clipped GRPO objective. `logp`, `old_logp`, `ref_logp`: [G, T] per-token log-probabilities of
    the sampled responses; `advantages`: [G] (one per response, from `GrpoGroup.advantages`);
    `mask`: [G, T] of valid tokens. The KL term is the unbiased k3 estimator exp(d) - d - 1 with
    d = ref_logp - logp."""
    adv = advantages.reshape(-1, 1).to(logp.dtype)
    ratio = torch.exp(logp - old_logp.detach())
    surr = torch.minimum(ratio * adv, torch.clamp(ratio, 1.0 - clip_eps, 1.0 + clip_eps) * adv)
    per_tok = -surr
    if ref_logp is not None and kl_coeff != 0.0:
        d = ref_logp.detach() - logp
        per_tok = per_tok + kl_coeff * (torch.exp(d) - d - 1.0)
    if mask is None:
        return per_tok.mean()
    m = mask.to(per_tok.dtype)
    return ((per_tok * m).sum(-1) / m.sum(-1).clamp_min(1.0)).mean()


class GrpoTrainer:
    def __init__(self, config: Optional[GrpoConfig] = None, verbose: bool = False):
        self.config = config or GrpoConfig()
        self.history: List[GrpoStats] = []
        self.verbose = verbose

    def step(self, groups: Sequence[GrpoGroup]) -> List[GrpoStats]:
        out = []
        for step, g in enumerate(groups):
            adv = g.advantages()
            n = max(len(g.rewards), 1)
            mean_r = sum(g.rewards) / n
            std_r = math.sqrt(sum((r - mean_r) ** 2 for r in g.rewards) / n)
            st = GrpoStats(step, mean_r, std_r, sum(adv) / max(len(adv), 1),
                           max(g.rewards, default=-math.inf), min(g.rewards, default=math.inf))
            if self.verbose and step % 10 == 0:
                print(f"  GRPO step {step}: mean_r={st.mean_reward:.3f} std_r={st.std_reward:.3f} "
                      f"best={st.best_reward:.3f} worst={st.worst_reward:.3f}")
            out.append(st)
        self.history.extend(out)
        return out

    def policy_step(self, policy_logp_fn, optimizer, groups: Sequence[GrpoGroup], old_logps, ref_logps=None, masks=None):
        """One optimisation pass over `groups`: `policy_logp_fn(group)` returns the [G, T] log-probs
        of the group's responses under the current policy. Returns the mean loss (a device tensor)."""
        total = None
        for it in range(self.config.num_iterations):
            for i, g in enumerate(groups):
                optimizer.zero_grad()
                logp = policy_logp_fn(g)
                adv = torch.tensor(g.advantages(), device=logp.device, dtype=logp.dtype)
                loss = grpo_loss(logp, old_logps[i], adv, None if ref_logps is None else ref_logps[i],
                                 self.config.clip_eps, self.config.kl_coeff, None if masks is None else masks[i])
                loss.backward()
                optimizer.step()
                total = loss.detach() if total is None else total + loss.detach()
        self.step(groups)
        return total / max(len(groups) * self.config.num_iterations, 1) if total is not None else None


# ------------------------------------------------------------------ reward model
class RewardDimension(enum.Enum):
    Correctness = 0
    Readability = 1
    Style = 2
    Aesthetics = 3


@dataclasses.dataclass
class RewardWeights:
    correctness: float = 0.5
    readability: float = 0.2
    style: float = 0.15
    aesthetics: float = 0.15


@dataclasses.dataclass
class RewardScore:
    correctness: float
    readability: float
    style: float
    aesthetics: float

    def total(self, w: RewardWeights) -> float:
        return (w.correctness * self.correctness + w.readability * self.readability
                + w.style * self.style + w.aesthetics * self.aesthetics)

    def to_vec(self) -> List[float]:
        return [self.correctness, self.readability, self.style, self.aesthetics]


def _clamp01(x: float) -> float:
    return min(max(x, 0.0), 1.0)


def _rust_lines(s: str) -> List[str]:
    """`str::lines`: split on '\\n', drop one trailing empty piece, strip a trailing '\\r'."""
    parts = s.split("\n")
    if parts and parts[-1] == "":
        parts.pop()
    return [p[:-1] if p.endswith("\r") else p for p in parts]


class RewardModel:
    """Heuristic code scorer (src/grpo.rs:215-420): each dimension is a sum of fixed bonuses."""

    def __init__(self, weights: Optional[RewardWeights] = None):
        self.weights = weights or RewardWeights()

    def score(self, code: str, tests_passed: Optional[bool] = None) -> RewardScore:
        return RewardScore(self._correctness(code, tests_passed), self._readability(code),
                           self._style(code), self._aesthetics(code))

    def reward(self, code: str, tests_passed: Optional[bool] = None) -> float:
        return self.score(code, tests_passed).total(self.weights)

    @staticmethod
    def _correctness(code: str, tests_passed: Optional[bool]) -> float:
        if tests_passed is not None:
            return 1.0 if tests_passed else 0.0
        s = 0.5
        if code.count("{") == code.count("}"):
            s += 0.2
        if "return" in code or "fn " in code:
            s += 0.15
        if "todo!" not in code and "unimplemented!" not in code:
            s += 0.15
        return _clamp01(s)

    @staticmethod
    def _readability(code: str) -> float:
        lines = _rust_lines(code)
        if not lines:
            return 0.0
        s = 0.0
        avg = sum(len(l.encode()) for l in lines) / len(lines)
        if 0.0 < avg < 100.0:
            s += 0.3
        fn_count = code.count("fn ")
        snake = sum(1 for l in lines if "fn " in l and not any(c.isupper() for c in l))
        s += 0.3 * (snake / fn_count) if fn_count > 0 else 0.3
        if any(l.lstrip().startswith("//") for l in lines):
            s += 0.2
        depth = mx = 0
        for c in code:
            if c == "{":
                depth += 1
            elif c == "}":
                depth -= 1
            mx = max(mx, depth)
        if mx <= 4:
            s += 0.2
        return _clamp01(s)

    @staticmethod
    def _style(code: str) -> float:
        lines = [l for l in _rust_lines(code) if l.strip()]
        if not lines:
            return 0.5
        s = 0.5
        units = {(len(l) - len(l.lstrip())) % 4 for l in lines if len(l) - len(l.lstrip()) > 0}
        if len(units) <= 1:
            s += 0.3
        if not any(l.endswith(" ") or l.endswith("\t") for l in _rust_lines(code)):
            s += 0.2
        return _clamp01(s)

    @staticmethod
    def _aesthetics(code: str) -> float:
        all_lines = _rust_lines(code)
        lines, non_empty = len(all_lines), sum(1 for l in all_lines if l.strip())
        if non_empty == 0:
            return 0.0
        s = 0.0
        nbytes = len(code.encode())
        if nbytes / non_empty < 80.0:
            s += 0.4
        comment = sum(len(l.encode()) for l in all_lines if l.lstrip().startswith("//"))
        if comment / max(nbytes, 1) < 0.3:
            s += 0.3
        if (lines - non_empty) / max(lines, 1) < 0.2:
            s += 0.3
        return _clamp01(s)


# ------------------------------------------------------------------ adversarial co-evolution
class ModelRole(enum.Enum):
    CodeGenerator = 0
    TestGenerator = 1


@dataclasses.dataclass
class AdversarialEpisode:
    problem: str
    generated_code: str
    generated_tests: str
    tests_passed: bool
    code_reward: RewardScore
    test_reward: float


@dataclasses.dataclass
class CoEvolutionStats:
    round: int
    code_pass_rate: float
    test_break_rate: float
    avg_code_reward: float
    difficulty: float


class CoEvolutionTrainer:
    """Code generator vs test generator (src/grpo.rs:459-590): code is rewarded by the reward model
    given the test verdict, tests by the fraction of code samples they break; both feed GRPO."""

    def __init__(self, grpo_config: Optional[GrpoConfig] = None, reward_weights: Optional[RewardWeights] = None, verbose: bool = False):
        self.config = grpo_config or GrpoConfig()
        self.grpo = GrpoTrainer(dataclasses.replace(self.config))
        self.reward_model = RewardModel(reward_weights)
        self.round = 0
        self.stats: List[CoEvolutionStats] = []
        self.verbose = verbose

    def co_evolve_round(self, problems: Sequence[str], code_samples: Dict[str, List[str]],
                        test_samples: Dict[str, List[str]], test_results: Sequence[Tuple[str, str, bool]]) -> List[AdversarialEpisode]:
        self.round += 1
        episodes: List[AdversarialEpisode] = []
        code_groups, test_groups = [], []
        passes = breaks = 0
        total_reward = 0.0
        for problem in problems:
            codes = list(code_samples.get(problem, []))
            tests = list(test_samples.get(problem, []))
            if not codes:
                continue
            rewards = []
            for i, code in enumerate(codes):
                passed = any(p == problem and ci == str(i) and ok for p, ci, ok in test_results)
                sc = self.reward_model.score(code, passed)
                rewards.append(sc.total(self.reward_model.weights))
                total_reward += rewards[-1]
                if passed:
                    passes += 1
                else:
                    breaks += 1
                episodes.append(AdversarialEpisode(problem, code, tests[0] if tests else "", passed, sc, 0.0 if passed else 1.0))
            code_groups.append(GrpoGroup(problem, codes, rewards))
            if tests:
                fails = sum(1 for p, _, ok in test_results if p == problem and not ok)
                test_groups.append(GrpoGroup(problem, tests, [fails / max(len(codes), 1)] * len(tests)))
        self.grpo.step(code_groups)
        self.grpo.step(test_groups)
        n = max(len(episodes), 1)
        st = CoEvolutionStats(self.round, passes / n, breaks / n, total_reward / n, self.round * 0.1)
        if self.verbose:
            print(f"  Co-evolution round {st.round}: pass_rate={st.code_pass_rate * 100:.1f}% "
                  f"break_rate={st.test_break_rate * 100:.1f}% avg_reward={st.avg_code_reward:.3f}")
        self.stats.append(st)
        return episodes


# ------------------------------------------------------------------ repository graph
@dataclasses.dataclass
class FileNode:
    path: str
    imports: List[str] = dataclasses.field(default_factory=list)
    exports: List[str] = dataclasses.field(default_factory=list)
    dependencies: List[str] = dataclasses.field(default_factory=list)


class StructureEdgeType(enum.Enum):
    Calls = 0
    Contains = 1
    Implements = 2
    References = 3


@dataclasses.dataclass
class StructureEdge:
    from_: str
    to: str
    edge_type: StructureEdgeType


class RepoGraph:
    def __init__(self):
        self.files: Dict[str, FileNode] = {}
        self.structure_edges: List[StructureEdge] = []
        self.functions: Set[str] = set()
        self.types: Set[str] = set()

    def add_file(self, node: FileNode) -> None:
        self.functions.update(node.exports)
        self.files[node.path] = node

    def add_edge(self, edge: StructureEdge) -> None:
        self.functions.add(edge.from_)
        self.functions.add(edge.to)
        self.structure_edges.append(edge)

    def dependents(self, path: str) -> List[str]:
        return [p for p, n in self.files.items() if path in n.imports]

    def dependencies(self, path: str) -> List[str]:
        n = self.files.get(path)
        return list(n.imports) if n else []

    def called_functions(self, func: str) -> List[str]:
        return [e.to for e in self.structure_edges if e.from_ == func and e.edge_type == StructureEdgeType.Calls]

    def context_for_file(self, path: str) -> List[str]:
        ctx: Set[str] = set()
        n = self.files.get(path)
        if n:
            for imp in n.imports:
                if imp in self.files:
                    ctx.update(self.files[imp].exports)
        for other in self.files.values():
            if path in other.imports:
                ctx.update(other.exports)
        return sorted(ctx)

    def circular_dependencies(self) -> List[List[str]]:
        cycles: List[List[str]] = []
        for start in self.files:
            visited: Set[str] = set()
            stack: List[str] = []
            self._dfs(start, visited, stack, cycles)
        return cycles

    def _dfs(self, node, visited, stack, cycles):
        if node in stack:
            cycles.append(stack[stack.index(node):])
            return
        if node in visited:
            return
        visited.add(node)
        stack.append(node)
        nd = self.files.get(node)
        if nd:
            for dep in nd.imports:
                self._dfs(dep, visited, stack, cycles)
        stack.pop()

    def num_files(self) -> int:
        return len(self.files)

    def num_edges(self) -> int:
        return len(self.structure_edges)

    def summary(self) -> str:
        return (f"RepoGraph: {self.num_files()} files, {len(self.functions)} functions, "
                f"{len(self.types)} types, {self.num_edges()} structural edges")


def _ident_pieces(s: str) -> List[str]:
    out, cur = [], []
    for c in s:
        if c.isalnum() or c == "_":
            cur.append(c)
        else:
            out.append("".join(cur)); cur = []
    out.append("".join(cur))
    return out


def parse_rust_file(path: str, source: str) -> FileNode:
    """Line-based scan of a Rust source (src/grpo.rs:770-830): `use` lines give external crates
    (first path segment unless crate/self) and internal imports (`crate::m` -> `src/m.rs`);
    `pub fn` / `pub async fn` / `pub struct` / `pub enum` lines give exports."""
    node = FileNode(path)
    for line in _rust_lines(source):
        t = line.strip()
        if t.startswith("use "):
            crate = t[4:].split("::")[0]
            if not crate.startswith("crate") and not crate.startswith("self"):
                node.dependencies.append(crate)
            if "crate::" in t:
                ws = t.split()
                parts = (ws[1] if len(ws) > 1 else "").rstrip(";").split("::")
                if len(parts) >= 2:
                    node.imports.append(f"src/{parts[1]}.rs")
        if t.startswith("pub fn ") or t.startswith("pub async fn "):
            ws = t.split("(")[0].split()
            k = 3 if t.startswith("pub async fn ") else 2      # the reference takes word 2 for both and so exports "fn" for async
            name = ws[k] if len(ws) > k else ""
            if name:
                node.exports.append(name)
        if t.startswith("pub struct ") or t.startswith("pub enum "):
            name = next((p for p in _ident_pieces(t) if p and p not in ("pub", "struct", "enum")), "")
            if name:
                node.exports.append(name)
    return node


from ._compat import install as _install  # noqa: E402

_install(globals())

from ._compat import alias_fields as _alias_fields  # noqa: E402

_alias_fields(StructureEdge, **{"from": "from_"})                          # `from` is a keyword here: getattr(edge, "from")
