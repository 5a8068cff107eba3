"""CPU tests of the training-recipe modules: GRPO / reward model / repo graph, RL agents and
environments, distillation, LoRA + schedules, self-improvement, diffusion, reasoning wrappers, MoE
(reference path), message framing, the TCP store and host-side failure detection."""
import math
import threading
import time

import pytest
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200 import grpo, rl, distill, finetune, self_improve, distributed as dist
from rust_neural_network_b200.loss import CrossEntropyLoss, MSELoss
from rust_neural_network_b200.models import diffusion, reasoning, moe
from rust_neural_network_b200.optim import Adam, SGD


# ------------------------------------------------------------------ GRPO
def test_grpo_advantages_and_best():
    g = grpo.GrpoGroup("p", ["a", "b", "c", "d"], [0.1, 0.2, 0.8, 0.9])
    adv = g.advantages()
    assert abs(sum(adv) / 4) < 1e-6
    assert abs(math.sqrt(sum(a * a for a in adv) / 4) - 1.0) < 1e-2
    g2 = grpo.GrpoGroup("p", ["bad", "good", "ok"], [0.1, 0.9, 0.5])
    assert g2.best_index() == 1 and g2.best_response() == "good"
    assert grpo.GrpoGroup("p", [], []).advantages() == []
    same = grpo.GrpoGroup("p", ["a", "b"], [0.5, 0.5]).advantages()
    assert all(abs(a) < 1e-3 for a in same)


def test_grpo_trainer_stats_and_loss():
    tr = grpo.GrpoTrainer(grpo.GrpoConfig())
    st = tr.step([grpo.GrpoGroup("t", ["a", "b"], [0.3, 0.7])])
    assert len(st) == 1 and st[0].best_reward > st[0].worst_reward and len(tr.history) == 1
    assert abs(st[0].mean_reward - 0.5) < 1e-6 and abs(st[0].std_reward - 0.2) < 1e-6
    # the clipped objective: a zero-advantage group has zero policy gradient, a positive one pushes logp up
    logp = torch.zeros(2, 3, requires_grad=True)
    old = torch.zeros(2, 3)
    loss = grpo.grpo_loss(logp, old, torch.tensor([1.0, -1.0]), ref_logp=old, clip_eps=0.2, kl_coeff=0.04)
    loss.backward()
    assert (logp.grad[0] < 0).all() and (logp.grad[1] > 0).all()
    # outside the clip range the gradient of the favoured sample vanishes
    logp2 = torch.full((1, 1), 0.5, requires_grad=True)
    grpo.grpo_loss(logp2, torch.zeros(1, 1), torch.tensor([1.0]), None, 0.2, 0.0).backward()
    assert float(logp2.grad.abs().sum()) == 0.0


def test_reward_model_heuristics():
    m = grpo.RewardModel()
    assert m.score("fn main() {}", True).correctness == 1.0
    assert m.score("fn main() {}", False).correctness == 0.0
    good = m.score("// adds\nfn add(a: i32, b: i32) -> i32 {\n    return a + b;\n}\n")
    bad = m.score("fn Foo( {{{ todo!()  \n\t x")
    assert good.correctness == pytest.approx(1.0) and bad.correctness < good.correctness
    assert good.readability == pytest.approx(1.0) and good.style == pytest.approx(1.0)
    assert 0.0 <= bad.style <= 1.0 and bad.style < good.style
    assert m.reward("fn a() {}", True) > m.reward("fn a() {}", False)
    assert m.score("").readability == 0.0 and m.score("").aesthetics == 0.0 and m.score("").style == 0.5
    w = grpo.RewardWeights()
    assert abs(w.correctness + w.readability + w.style + w.aesthetics - 1.0) < 1e-6
    assert len(good.to_vec()) == 4


def test_co_evolution_round():
    tr = grpo.CoEvolutionTrainer()
    eps = tr.co_evolve_round(["p1"], {"p1": ["fn a() {}", "fn b() { todo!() }"]}, {"p1": ["#[test] fn t() {}"]},
                             [("p1", "0", True), ("p1", "1", False)])
    assert len(eps) == 2 and eps[0].tests_passed and not eps[1].tests_passed
    assert eps[1].test_reward == 1.0 and eps[0].test_reward == 0.0
    st = tr.stats[-1]
    assert st.round == 1 and st.code_pass_rate == 0.5 and st.test_break_rate == 0.5 and abs(st.difficulty - 0.1) < 1e-9
    assert len(tr.grpo.history) == 2
    assert tr.co_evolve_round(["zz"], {}, {}, []) == []


def test_repo_graph_and_parser():
    src = "use std::collections::HashMap;\nuse crate::tensor::Tensor;\nuse self::x;\npub fn forward(x: &Tensor) -> Tensor {\n}\npub struct Layer<T> {\n}\npub enum Kind {\nfn private() {}\npub async fn go() {}\n"
    n = grpo.parse_rust_file("src/nn.rs", src)
    assert n.dependencies == ["std"] and n.imports == ["src/tensor.rs"]
    assert n.exports == ["forward", "Layer", "Kind", "go"]
    g = grpo.RepoGraph()
    g.add_file(n)
    g.add_file(grpo.FileNode("src/tensor.rs", imports=["src/nn.rs"], exports=["Tensor"]))
    g.add_file(grpo.FileNode("src/lone.rs"))
    assert g.num_files() == 3 and g.dependents("src/tensor.rs") == ["src/nn.rs"] and g.dependencies("src/nn.rs") == ["src/tensor.rs"]
    assert g.context_for_file("src/nn.rs") == ["Tensor"]
    cyc = g.circular_dependencies()
    assert any(set(c) == {"src/nn.rs", "src/tensor.rs"} for c in cyc)
    g.add_edge(grpo.StructureEdge("forward", "matmul", grpo.StructureEdgeType.Calls))
    g.add_edge(grpo.StructureEdge("Layer", "Module", grpo.StructureEdgeType.Implements))
    assert g.called_functions("forward") == ["matmul"] and g.called_functions("Layer") == [] and g.num_edges() == 2
    assert g.summary().startswith("RepoGraph: 3 files")


# ------------------------------------------------------------------ RL
def test_rl_helpers_and_envs():
    assert rl.discounted_returns([1.0, 1.0, 1.0], 0.5) == pytest.approx([1.75, 1.5, 1.0])
    counts = [0, 0]
    import random
    rng = random.Random(0)
    for _ in range(400):
        counts[rl.sample_categorical([0.0, 2.0], rng)] += 1
    assert counts[1] > counts[0] * 3
    env = rl.ChainEnv.new(4)
    obs = env.reset()
    assert len(obs) == 4 and obs[3] == 1.0 and env.num_actions() == 2 and env.observation_dim() == 4
    done, total = False, 0.0
    while not done:
        obs, r, done = env.step(0)
        total += r
    assert total > 0
    b = rl.BanditEnv.sparse(3)
    b.reset()
    assert b.step(0)[1] == 1.0 and b.step(1)[1] == 0.0 and b.num_actions() == 3
    assert rl.clipped_advantage_weight(1.0, 0.0, 1.0, 0.2) == 0.0 and rl.clipped_advantage_weight(1.0, 0.0, 0.1, 0.2) == 1.0
    assert rl.clipped_advantage_weight(-1.0, 0.0, -1.0, 0.2) == 0.0 and rl.clipped_advantage_weight(-1.0, 0.0, 1.0, 0.2) == -1.0


def test_replay_buffer_ring():
    buf = rl.ReplayBuffer.with_seed(3, 1)
    assert buf.is_empty()
    for i in range(5):
        buf.push(rl.Transition([float(i)], 0, float(i), [0.0], False))
    assert buf.len() == 3 and sorted(t.reward for t in buf.data) == [2.0, 3.0, 4.0]
    assert len(buf.sample(2)) == 2


def test_reinforce_learns_bandit():
    torch.manual_seed(0)
    env = rl.BanditEnv.sparse(3)
    agent = rl.Reinforce(1, 3, 8)
    opt = Adam(agent.parameters(), lr=0.05)
    for _ in range(60):
        agent.train_episode(opt, env)
    logits = agent.policy(torch.tensor([[1.0]])).detach()[0]
    assert int(logits.argmax()) == 0


def test_actor_critic_dqn_ppo_run():
    torch.manual_seed(0)
    env = rl.ChainEnv.with_max_steps(4, 20)
    ac = rl.ActorCritic(4, 2, 8)
    r = ac.train_episode(Adam(ac.parameters(), lr=0.01), env)
    assert math.isfinite(r)
    dqn = rl.Dqn.with_seed(4, 2, 8, 3)
    buf = rl.ReplayBuffer.with_seed(64, 2)
    obs = env.reset()
    for _ in range(32):
        a = dqn.act(obs)
        nxt, rew, done = env.step(a)
        buf.push(rl.Transition(obs, a, rew, nxt, done))
        obs = env.reset() if done else nxt
    loss = dqn.train_step(buf, Adam(dqn.parameters(), lr=0.01), 16)
    assert loss is None or math.isfinite(float(loss))
    dqn.sync_target()
    ppo = rl.Ppo(4, 2, 8)
    out = ppo.update(env, 16, Adam(ppo.parameters(), lr=0.01))
    assert math.isfinite(out)


# ------------------------------------------------------------------ distill / finetune / self-improve
def _toy_classification(n=64, d=6, c=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, d, generator=g)
    w = torch.randn(d, c, generator=g)
    return x, (x @ w).argmax(-1)


def test_distiller_student_shape_and_learning():
    torch.manual_seed(0)
    x, y = _toy_classification()
    teacher = nn.Sequential().add(nn.Linear(6, 64)).add(nn.ReLU()).add(nn.Linear(64, 64)).add(nn.ReLU()).add(nn.Linear(64, 64)).add(nn.ReLU()).add(nn.Linear(64, 3))
    topt = Adam(teacher.parameters(), lr=0.01)
    ce = CrossEntropyLoss()
    for _ in range(60):
        topt.zero_grad(); l = ce(teacher(x), y); l.backward(); topt.step()
    d = distill.Distiller(teacher, distill.DistillConfig(epochs=30, lr=0.01, batch_size=32))
    student = d.generate_student(6, 3)
    shapes = [tuple(p.shape) for p in student.parameters() if p.dim() == 2]
    assert shapes == [(32, 6), (3, 32)]
    res = d.distill(x, y, 6, 3)
    assert res.compression_ratio > 1.0 and res.loss_history[-1] < res.loss_history[0]
    assert res.student_accuracy > 0.6 and res.teacher_accuracy > 0.8
    p = distill.softmax_temp(torch.tensor([[1.0, 2.0, 3.0]]), 4.0)
    assert float(p.sum()) == pytest.approx(1.0) and float(p.max()) < float(torch.softmax(torch.tensor([1.0, 2.0, 3.0]), -1).max())
    prog = distill.ProgressiveDistiller(distill.DistillConfig(epochs=2), 2).distill(teacher, x, y, 6, 3)
    assert len(prog) == 2


def test_lora_and_schedules():
    torch.manual_seed(0)
    lin = nn.Linear(5, 4)
    ad = finetune.LoraAdapter.from_linear(lin, 2, 4.0)
    x = torch.randn(3, 5)
    assert torch.allclose(ad(x), lin(x), atol=1e-5)                 # B = 0 -> adapter is the identity on top of W
    assert float(ad.weight_delta().abs().sum()) == 0.0 and ad.scale == 2.0
    ad.lora_b.data.normal_()
    want = x @ ad.merge().T + lin.bias.detach()
    assert torch.allclose(ad(x), want, atol=1e-4)
    ad(x).sum().backward()
    assert ad.lora_a.grad is not None and ad.lora_b.grad is not None and ad.frozen_weight.grad is None
    assert len(ad.trainable_parameters()) == 2
    s = finetune.LrSchedule.CosineWithWarmup(10, 110, 1.0, 0.1)
    assert s.lr(0) == 0.0 and s.lr(5) == pytest.approx(0.5) and s.lr(10) == pytest.approx(1.0)
    assert s.lr(60) == pytest.approx(0.55) and s.lr(110) == pytest.approx(0.1)
    assert finetune.LrSchedule.Constant().lr(7) == 0.001
    assert finetune.LrSchedule.Warmup(4, 2.0).lr(2) == pytest.approx(1.0) and finetune.LrSchedule.Warmup(4, 2.0).lr(9) == 2.0
    assert finetune.FastTrainConfig().with_accum(4).effective_batch_size() == 128


def test_fast_trainer_accumulates_and_clips():
    from rust_neural_network_b200.train import SimpleDataLoader
    torch.manual_seed(0)
    x, y = _toy_classification(64)
    model = nn.Sequential().add(nn.Linear(6, 16)).add(nn.ReLU()).add(nn.Linear(16, 3))
    cfg = finetune.FastTrainConfig(epochs=8, micro_batch_size=8, grad_accum_steps=2, log_every=1,
                                   lr_schedule=finetune.LrSchedule.Warmup(2, 0.02))
    tr = finetune.FastTrainer(model, cfg)
    hist = tr.fit(SimpleDataLoader(x, y, 8), Adam(model.parameters(), lr=0.02), CrossEntropyLoss())
    assert tr.total_steps() == 8 * 4 and len(hist) == 32
    assert hist[-1].loss < hist[0].loss and hist[0].lr == 0.0 and hist[-1].lr == pytest.approx(0.02)
    p = [torch.nn.Parameter(torch.ones(4))]
    p[0].grad = torch.full((4,), 3.0)
    assert finetune.clip_grad_norm(p, 1.0) == pytest.approx(6.0) and float(p[0].grad.norm()) == pytest.approx(1.0, abs=1e-4)


def test_self_improver_runs():
    torch.manual_seed(0)

    class NormCritic(self_improve.Critic):
        def evaluate(self, inp, out):
            return float(1.0 / (1.0 + out.detach().float().pow(2).mean()))
    model = nn.Sequential().add(nn.Linear(4, 4))
    imp = self_improve.SelfImprover(model, SGD(model.parameters(), lr=0.05), NormCritic(), 0.0)
    xs = [torch.randn(2, 4) for _ in range(4)]
    r0 = imp.self_train_epoch(xs)
    for _ in range(5):
        r1 = imp.self_train_epoch(xs)
    assert math.isfinite(r0) and math.isfinite(r1)


# ------------------------------------------------------------------ diffusion / reasoning
def test_noise_schedule_and_ddpm():
    torch.manual_seed(0)
    for kind in (diffusion.ScheduleType.Linear, diffusion.ScheduleType.Cosine):
        s = diffusion.NoiseSchedule.new(kind, 50)
        ac = torch.as_tensor(s.alpha_cumprod)
        assert ac.numel() == 50 and bool((ac[1:] <= ac[:-1] + 1e-7).all()) and 0 < float(ac[-1]) < float(ac[0]) <= 1.0
    m = diffusion.DDPM(4, 16, 20)
    x0 = torch.randn(8, 4) * 0.1 + 1.0
    noise = torch.randn(8, 4)
    xt = m.q_sample(x0, 5, noise)
    ac = float(torch.as_tensor(m.schedule.alpha_cumprod)[5])
    assert torch.allclose(xt, math.sqrt(ac) * x0 + math.sqrt(1 - ac) * noise, atol=1e-5)
    opt = Adam(m.parameters(), lr=0.01)
    l0 = sum(m.train_batch(opt, x0) for _ in range(5)) / 5
    for _ in range(60):
        m.train_batch(opt, x0)
    l1 = sum(m.train_batch(opt, x0) for _ in range(5)) / 5
    assert l1 < l0
    out = m.sample(3)
    assert tuple(out.shape) == (3, 4) and bool(torch.isfinite(out).all())


def test_reasoning_wrappers_shapes_and_grads():
    torch.manual_seed(0)
    x = torch.randn(3, 8)
    for mod in (reasoning.ChainOfThought(8, 3), reasoning.ChainOfThought(8, 2).with_residual(True),
                reasoning.TreeOfThoughts(8, 2, 2, 2), reasoning.SwiReasoning(8, 3, 0.5), reasoning.MarkovianRSA(8, 3, 2)):
        y = mod(x)
        assert tuple(y.shape) == (3, 8) and bool(torch.isfinite(y).all())
        if isinstance(mod, reasoning.MarkovianRSA):      # its aggregation layer is a parameter but not on the path
            assert torch.allclose(y, 3 * x, atol=1e-5) and len(mod.parameters()) == 2
            continue
        y.float().pow(2).sum().backward()
        assert any(p.grad is not None and float(p.grad.abs().sum()) > 0 for p in mod.parameters())


# ------------------------------------------------------------------ MoE (reference path on CPU)
def test_moe_router_ref_and_layers_cpu():
    torch.manual_seed(0)
    logits = torch.randn(10, 4)
    idx, w, probs = moe.router_ref(logits, 2, True)
    assert tuple(idx.shape) == (10, 2) and torch.allclose(w.sum(-1), torch.ones(10), atol=1e-5)
    assert torch.allclose(probs.sum(-1), torch.ones(10), atol=1e-5)
    top = torch.softmax(logits, -1).topk(2, -1).indices
    assert torch.equal(idx.long().sort(-1).values, top.sort(-1).values)
    layer = moe.NormalMoE(6, 12, 4, top_k=2)
    x = torch.randn(5, 6)
    y = layer(x)
    assert tuple(y.shape) == (5, 6)
    (y.float().sum() + layer.last_aux_loss).backward()
    assert all(p.grad is not None for p in layer.parameters())
    fg = moe.FineGrainedMoE(6, 8, 4, 8, top_k=3)
    assert tuple(fg(x).shape) == (5, 6)


# ------------------------------------------------------------------ distributed host runtime
def test_message_framing_is_byte_exact():
    m = dist.Message.gradient_chunk([1.0, -2.5])
    b = m.serialize()
    assert b[0] == 0 and int.from_bytes(b[1:5], "little") == 8 and len(b) == 13
    back = dist.Message.deserialize(b)
    assert back.msg_type == dist.MessageType.GradientChunk and back.as_floats() == [1.0, -2.5]
    assert dist.Message.deserialize(b[:7]) is None and dist.Message.deserialize(bytes([9, 0, 0, 0, 0])) is None
    assert dist.Message.barrier().serialize() == bytes([1, 0, 0, 0, 0])


def test_ring_all_reduce_and_config():
    workers = [[1.0, 2.0, 3.0, 4.0, 5.0], [10.0, 20.0, 30.0, 40.0, 50.0], [100.0, 200.0, 300.0, 400.0, 500.0]]
    dist.ring_all_reduce_all(workers, 3)
    for w in workers:
        assert w == pytest.approx([111.0, 222.0, 333.0, 444.0, 555.0])
    d = [3.0, 6.0]
    dist.average_gradients(d, 3)
    assert d == pytest.approx([1.0, 2.0])
    c = dist.DistributedConfig.new(1, 4)
    assert c.shard_range(10) == (3, 6) or c.shard_range(10)[1] - c.shard_range(10)[0] in (2, 3)
    covered = []
    for r in range(4):
        a, b = dist.DistributedConfig.new(r, 4).shard_range(10)
        covered += list(range(a, b))
    assert covered == list(range(10))
    assert c.local_batch_size(64) == 16 and dist.DistributedConfig.single().world_size == 1


def test_flatten_sync_clip():
    p = [torch.nn.Parameter(torch.zeros(2, 2)), torch.nn.Parameter(torch.zeros(3))]
    p[0].grad = torch.ones(2, 2); p[1].grad = torch.full((3,), 2.0)
    flat = dist.flatten_gradients(p)
    assert flat.tolist() == [1, 1, 1, 1, 2, 2, 2]
    dist.sync_gradients(p, 2, [torch.full((7,), 3.0)], 0)
    assert p[0].grad.flatten().tolist() == [2.0] * 4 and p[1].grad.tolist() == [2.5] * 3
    n = dist.clip_gradients(p, 1.0)
    assert n == pytest.approx(math.sqrt(4 * 4 + 3 * 6.25), rel=1e-4)
    assert float(dist.flatten_gradients(p).norm()) == pytest.approx(1.0, abs=1e-4)


def test_tcp_store_set_get_add_barrier_timeout():
    master = dist.TcpStore(is_master=True)
    try:
        client = dist.TcpStore(port=master.port)
        master.set("k", b"hello")
        assert client.get("k", wait=1.0) == b"hello"
        assert client.add("n", 2) == 2 and master.add("n", 3) == 5
        t0 = time.time()
        assert client.get("absent", wait=0.2) is None           # a bounded wait that runs out
        assert time.time() - t0 < 3.0
        # a late set wakes a blocked get
        threading.Timer(0.1, lambda: master.set("late", b"x")).start()
        assert client.get("late", wait=3.0) == b"x"
        res = []
        th = threading.Thread(target=lambda: res.append(client.barrier("b", 2, 3.0)))
        th.start()
        assert master.barrier("b", 2, 3.0)
        th.join()
        assert res == [True]
        assert not master.barrier("lonely", 2, 0.2)              # a rank that never joins -> False, not a hang
        client.close()
    finally:
        master.close()


def test_heartbeat_detects_dead_rank():
    master = dist.TcpStore(is_master=True)
    try:
        c1 = dist.TcpStore(port=master.port)
        hb0 = dist.HeartbeatMonitor(master, 0, 2, interval=0.05, timeout=0.3).start()
        hb1 = dist.HeartbeatMonitor(c1, 1, 2, interval=0.05, timeout=0.3).start()
        time.sleep(0.2)
        assert hb0.dead_ranks() == []
        hb1.stop()                                                # rank 1 stops beating (host-side failure)
        deadline = time.time() + 3.0
        dead = []
        while time.time() < deadline and not dead:
            time.sleep(0.1)
            dead = hb0.dead_ranks()
        assert dead == [1]
        hb0.stop(); c1.close()
    finally:
        master.close()


def test_distributed_worker_standalone_step_and_rendezvous_timeout():
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(3, 2))
    w = dist.DistributedWorker.standalone(0, 1)
    x, y = torch.randn(4, 3), torch.randn(4, 2)
    l0 = w.train_step(model, SGD(model.parameters(), lr=0.1), MSELoss(), x, y)
    for _ in range(10):
        l1 = w.train_step(model, SGD(model.parameters(), lr=0.1), MSELoss(), x, y)
    assert l1 < l0
    with pytest.raises(TimeoutError):
        dist.DistributedWorker.connect(0, 2, master_port=0, timeout=0.3)   # the peer never joins


def test_split_cols_backward_fills_one_buffer():
    """The (x, z) split of a fused projection: views forward, both gradients written into one matrix backward; a missing
    gradient becomes zeros."""
    from rust_neural_network_b200.parallel.tp import split_cols
    x = torch.randn(6, 10, requires_grad=True)
    a, b = split_cols(x, 4)
    assert a.shape == (6, 4) and b.shape == (6, 6) and a.data_ptr() == x.data_ptr()
    ga, gb = torch.randn(6, 4), torch.randn(6, 6)
    (a * ga).sum().backward(retain_graph=True)
    assert torch.equal(x.grad[:, :4], ga) and float(x.grad[:, 4:].abs().sum()) == 0.0
    x.grad = None
    ((a * ga).sum() + (b * gb).sum()).backward()
    assert torch.equal(x.grad, torch.cat([ga, gb], 1))


def test_rows2d_accepts_column_slices_and_collapsible_batches():
    from rust_neural_network_b200.ops.kernels import _rows2d
    wide = torch.zeros(4, 6, 32)
    t, rows, cols, ld = _rows2d(wide[:, :, 16:])                    # a column slice: rows 32 apart
    assert (rows, cols, ld) == (24, 16, 32) and t.data_ptr() == wide[:, :, 16:].data_ptr()
    t, rows, cols, ld = _rows2d(wide[:, ::2, :16])                  # every other row: still one row stride
    assert (rows, cols, ld) == (12, 16, 64)
    t, rows, cols, ld = _rows2d(wide.transpose(0, 1)[:, :, :16])    # batches that do not collapse: copied
    assert (rows, cols, ld) == (24, 16, 16) and t.is_contiguous()
    t, rows, cols, ld = _rows2d(torch.zeros(8, 5).t())              # no unit inner stride: copied
    assert (rows, cols, ld) == (5, 8, 8)
