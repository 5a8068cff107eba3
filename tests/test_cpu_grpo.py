"""grpo.py, one test per behaviour of rust-nn src/grpo.rs:835-1080: group-relative advantages, the best response, the
trainer's statistics, the four reward dimensions and their weighted total, the repository graph (context, dependencies,
call edges, Rust source parsing, summary) and a co-evolution round."""
import math

from rust_neural_network_b200 import grpo as G


def test_advantages_are_zero_mean():
    adv = G.GrpoGroup("test", ["a", "b", "c"], [1.0, 2.0, 3.0]).advantages()
    assert abs(sum(adv) / len(adv)) < 1e-5


def test_advantages_have_unit_std():
    adv = G.GrpoGroup("test", ["a", "b", "c", "d"], [0.1, 0.2, 0.8, 0.9]).advantages()
    assert abs(math.sqrt(sum(a * a for a in adv) / len(adv)) - 1.0) < 0.01


def test_equal_rewards_give_zero_advantages_not_nan():
    adv = G.GrpoGroup("test", ["a", "b"], [0.5, 0.5]).advantages()
    assert adv == [0.0, 0.0]
    assert G.GrpoGroup("test", [], []).advantages() == []


def test_best_response():
    g = G.GrpoGroup("test", ["bad", "good", "ok"], [0.1, 0.9, 0.5])
    assert g.best_index() == 1 and g.best_response() == "good"


def test_trainer_tracks_stats():
    tr = G.GrpoTrainer(G.GrpoConfig())
    stats = tr.step([G.GrpoGroup("test", ["a", "b"], [0.3, 0.7])])
    assert len(stats) == 1 and stats[0].best_reward > stats[0].worst_reward
    assert abs(stats[0].mean_reward - 0.5) < 1e-6 and abs(stats[0].mean_advantage) < 1e-5
    assert tr.step([G.GrpoGroup("t", ["a"], [1.0])])[0].step == 0        # the index within the call, as the reference numbers it
    assert len(tr.history) == 2


def test_reward_correctness_follows_the_test_verdict():
    m = G.RewardModel(G.RewardWeights())
    assert abs(m.score("fn main() {}", True).correctness - 1.0) < 1e-5
    assert abs(m.score("fn main() { panic!() }", False).correctness - 0.0) < 1e-5


def test_reward_readability_of_commented_well_named_code():
    code = "// Good function\nfn calculate_sum(a: i32, b: i32) -> i32 {\n    a + b\n}\n"
    assert G.RewardModel(G.RewardWeights()).score(code, None).readability > 0.5


def test_reward_aesthetics_prefers_concise_code():
    m = G.RewardModel(G.RewardWeights())
    concise = "fn add(a: i32, b: i32) -> i32 { a + b }\n"
    verbose = ("fn add(a: i32, b: i32) -> i32 {\n    // This function adds two numbers\n    // It takes two i32 parameters\n"
               "    // And returns their sum\n    let result = a + b;\n    return result;\n}\n")
    assert m.score(concise, None).aesthetics >= m.score(verbose, None).aesthetics


def test_reward_total_is_the_weighted_sum():
    w = G.RewardWeights(correctness=0.5, readability=0.2, style=0.15, aesthetics=0.15)
    m = G.RewardModel(w)
    code = "fn add(a: i32, b: i32) -> i32 { a + b }\n"
    r = m.reward(code, True)
    assert r > 0.5
    s = m.score(code, True)
    assert abs(r - (0.5 * s.correctness + 0.2 * s.readability + 0.15 * s.style + 0.15 * s.aesthetics)) < 1e-6
    assert len(s.to_vec()) == 4


def test_repo_graph_context_lists_the_exports_of_imported_files():
    g = G.RepoGraph()
    g.add_file(G.FileNode("src/main.rs", ["src/lib.rs"], ["main"], []))
    g.add_file(G.FileNode("src/lib.rs", [], ["add", "subtract"], ["ndarray"]))
    ctx = g.context_for_file("src/main.rs")
    assert "add" in ctx and "subtract" in ctx
    assert g.dependents("src/lib.rs") == ["src/main.rs"]


def test_repo_graph_dependencies():
    g = G.RepoGraph()
    g.add_file(G.FileNode("src/a.rs", ["src/b.rs", "src/c.rs"], ["func_a"], []))
    assert len(g.dependencies("src/a.rs")) == 2
    assert g.dependencies("src/missing.rs") == []


def test_repo_graph_called_functions():
    g = G.RepoGraph()
    for a, b in (("func_a", "func_b"), ("func_a", "func_c"), ("func_b", "func_d")):
        g.add_edge(G.StructureEdge(a, b, G.StructureEdgeType.Calls))
    called = g.called_functions("func_a")
    assert sorted(called) == ["func_b", "func_c"]


def test_parse_rust_file_extracts_public_items():
    src = "\nuse crate::lib::helper;\n\npub fn calculate(x: i32) -> i32 { x * 2 }\npub struct Config { name: String }\nfn private_helper() {}\n"
    node = G.parse_rust_file("src/calc.rs", src)
    assert "calculate" in node.exports and "Config" in node.exports and "private_helper" not in node.exports
    assert "crate" in node.dependencies or "src/lib.rs" in node.imports


def test_repo_graph_summary_and_cycles():
    g = G.RepoGraph()
    g.add_file(G.FileNode("a.rs", [], ["f"], []))
    g.add_edge(G.StructureEdge("f", "g", G.StructureEdgeType.Calls))
    s = g.summary()
    assert "1 files" in s and "1 structural edges" in s
    assert g.num_files() == 1 and g.num_edges() == 1
    h = G.RepoGraph()
    h.add_file(G.FileNode("x.rs", ["y.rs"], [], []))
    h.add_file(G.FileNode("y.rs", ["x.rs"], [], []))
    assert h.circular_dependencies()


def test_co_evolution_round():
    tr = G.CoEvolutionTrainer(G.GrpoConfig(), G.RewardWeights())
    p = "write add function"
    episodes = tr.co_evolve_round([p], {p: ["fn add(a: i32, b: i32) -> i32 { a + b }", "fn add(a, b) { a + b }"]},
                                  {p: ["assert_eq!(add(1, 2), 3);"]}, [(p, "0", True), (p, "1", False)])
    assert episodes and len(tr.stats) == 1 and tr.stats[0].code_pass_rate > 0.0
    assert 0.0 <= tr.stats[0].test_break_rate <= 1.0
