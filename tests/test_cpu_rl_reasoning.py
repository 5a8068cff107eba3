"""Reinforcement-learning agents and the reasoning wrappers, one test per behaviour of rust-nn tests/rl.rs:10-240
and tests/reasoning.rs:14-125."""
import random

import torch

from rust_neural_network_b200 import rl
from rust_neural_network_b200.models.reasoning import ChainOfThought, TreeOfThoughts
from rust_neural_network_b200.optim import Adam


def _greedy(policy, obs):
    with torch.no_grad():
        return int(policy(torch.tensor([obs]))[0].argmax())


# ------------------------------------------------------------------ rl
def test_categorical_sample_respects_the_distribution():
    rng = random.Random(0)
    counts = [0, 0, 0]
    for _ in range(2000):
        counts[rl.sample_categorical([-10.0, -10.0, 10.0], rng)] += 1
    assert counts[2] > counts[0] + counts[1]


def test_discounted_returns():
    r = rl.discounted_returns([1.0, 2.0, 3.0], 0.5)
    assert [round(v, 5) for v in r] == [2.75, 3.5, 3.0]


def test_reinforce_learns_the_bandit():
    torch.manual_seed(0); random.seed(0)
    agent = rl.Reinforce(1, 4, 16)
    opt = Adam(agent.policy.parameters(), lr=0.02)
    env = rl.BanditEnv.sparse(4)
    for _ in range(300):
        agent.train_episode(opt, env)
    assert _greedy(agent.policy, [1.0]) == 0


def test_actor_critic_learns_the_bandit():
    torch.manual_seed(0); random.seed(0)
    agent = rl.ActorCritic(1, 4, 16)
    opt = Adam(agent.actor.parameters() + agent.critic.parameters(), lr=0.02)
    env = rl.BanditEnv.sparse(4)
    for _ in range(300):
        agent.train_episode(opt, env)
    assert _greedy(agent.actor, [1.0]) == 0


def test_ppo_learns_the_bandit():
    torch.manual_seed(0); random.seed(0)
    agent = rl.Ppo(1, 4, 16)
    opt = Adam(agent.actor.parameters() + agent.critic.parameters(), lr=0.02)
    env = rl.BanditEnv.sparse(4)
    for _ in range(60):
        agent.update(env, 64, opt)
    assert _greedy(agent.actor, [1.0]) == 0


def test_replay_buffer_keeps_the_newest():
    buf = rl.ReplayBuffer.new(4)
    assert buf.is_empty()
    for i in range(10):
        buf.push(rl.Transition([float(i)], i % 3, float(i), [float(i + 1)], i == 9))
    assert buf.len() == 4
    assert sorted(t.reward for t in buf.data) == [6.0, 7.0, 8.0, 9.0]
    assert len(buf.sample(2)) == 2


def test_dqn_reduces_its_td_error():
    torch.manual_seed(0)
    n = 4
    agent = rl.Dqn.with_seed(n, 2, 32, 42)
    opt = Adam(agent.parameters(), lr=0.01)
    buf = rl.ReplayBuffer.with_seed(8000, 7)
    env = rl.ChainEnv.with_max_steps(n, 16)
    agent.epsilon = 1.0
    for _ in range(150):                                            # random experience
        o, done = env.reset(), False
        while not done:
            a = agent.act(o)
            nxt, r, done = env.step(a)
            buf.push(rl.Transition(list(o), a, r, list(nxt), done))
            o = nxt
    probe = buf.sample(64)
    before = float(agent.td_error(probe).detach().abs().mean())
    agent.epsilon = 0.2
    for _ in range(300):
        agent.train_step(buf, opt, 32)
    after = float(agent.td_error(probe).detach().abs().mean())
    assert after < before


def test_dqn_sync_target_copies_the_online_weights():
    torch.manual_seed(0)
    agent = rl.Dqn.new(3, 2, 8)
    buf = rl.ReplayBuffer.new(100)
    for _ in range(20):
        buf.push(rl.Transition([1.0, 1.0, 1.0], 0, 5.0, [1.0, 1.0, 1.0], False))
    online_before = [p.detach().clone() for p in agent.q_net.parameters()]
    target_before = [p.detach().clone() for p in agent.target_net.parameters()]
    agent.train_step(buf, Adam(agent.parameters(), lr=0.1), 8)
    assert any(not torch.equal(a, b.detach()) for a, b in zip(online_before, agent.q_net.parameters()))
    assert all(torch.equal(a, b.detach()) for a, b in zip(target_before, agent.target_net.parameters()))
    agent.sync_target()
    assert all(torch.equal(a.detach(), b.detach()) for a, b in zip(agent.target_net.parameters(), agent.q_net.parameters()))
    assert any(not torch.equal(a, b.detach()) for a, b in zip(target_before, agent.target_net.parameters()))


# ------------------------------------------------------------------ reasoning
def test_cot_preserves_shape():
    assert list(ChainOfThought(8, 4)(torch.randn(3, 8)).shape) == [3, 8]


def test_cot_is_differentiable_through_the_whole_chain():
    x = torch.tensor([[0.5, -0.3, 0.8, -0.1, 0.2, -0.4]], requires_grad=True)
    ChainOfThought(6, 3)(x).sum().backward()
    assert bool((x.grad.abs() > 0).all())


def test_cot_with_zero_steps_is_the_identity():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.equal(ChainOfThought(4, 0)(x), x)


def test_cot_with_and_without_residual():
    x = torch.ones(1, 4)
    for cot in (ChainOfThought(4, 5), ChainOfThought(4, 5).with_residual(False)):
        y = cot(x)
        assert list(y.shape) == [1, 4] and bool(torch.isfinite(y).all())


def test_tot_preserves_shape():
    assert list(TreeOfThoughts(8, 3, 4, 2)(torch.randn(2, 8)).shape) == [2, 8]


def test_tot_with_exploration_noise():
    assert list(TreeOfThoughts(6, 4, 3, 2).with_exploration_noise(0.2)(torch.randn(1, 6)).shape) == [1, 6]


def test_tot_beam_width_one_is_greedy():
    y = TreeOfThoughts(5, 3, 3, 1)(torch.randn(2, 5))
    assert list(y.shape) == [2, 5] and bool(torch.isfinite(y).all())


def test_tot_without_noise_is_deterministic():
    tot = TreeOfThoughts(4, 2, 2, 1).with_exploration_noise(0.0)
    x = torch.randn(1, 4)
    y = tot(x)
    assert list(y.shape) == [1, 4] and torch.equal(y, tot(x))


def test_tot_has_thought_and_evaluator_parameters():
    assert len(TreeOfThoughts(8, 2, 2, 2).parameters()) >= 4
