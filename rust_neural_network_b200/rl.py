"""Reinforcement learning (rust-nn src/rl.rs): `Environment`, `Reinforce`, `ActorCritic`, `Dqn` (+
`ReplayBuffer`, `Transition`), `Ppo`, `BanditEnv`, `ChainEnv`, `sample_categorical`, `discounted_returns`.

Same networks, hyper-parameters and update rules as the reference. Where the reference loops over the
steps of an episode and calls `backward()` once per step (accumulating gradients), the episode is
stacked into one batch here and the summed loss is back-propagated once - the accumulated gradient is
identical, the work is one batched GEMM pass.
"""
from __future__ import annotations

import dataclasses
import math
import random
from typing import List, Sequence, Tuple

import torch

from . import nn


class Environment:
    def reset(self) -> List[float]: raise NotImplementedError
    def step(self, action: int) -> Tuple[List[float], float, bool]: raise NotImplementedError
    def observation_dim(self) -> int: raise NotImplementedError
    def num_actions(self) -> int: raise NotImplementedError


_rng = random.Random()


def sample_categorical(logits: Sequence[float], rng: random.Random = None) -> int:
    """Categorical sample from logits by the cumulative-distribution method (src/rl.rs:34-60)."""
    rng = rng or _rng
    m = max(logits)
    ex = [math.exp(x - m) for x in logits]
    s = sum(ex)
    u, acc = rng.random() * s, 0.0
    for i, e in enumerate(ex):
        acc += e
        if u <= acc:
            return i
    return len(logits) - 1


def discounted_returns(rewards: Sequence[float], gamma: float) -> List[float]:
    out, g = [0.0] * len(rewards), 0.0
    for t in reversed(range(len(rewards))):
        g = rewards[t] + gamma * g
        out[t] = g
    return out


def _policy(obs_dim, hidden, out, act):
    return nn.Sequential(nn.Linear(obs_dim, hidden), act(), nn.Linear(hidden, out))


def _obs(batch, device):
    return torch.tensor(batch, dtype=torch.float32, device=device)


def _logp(logits, actions):
    return torch.log_softmax(logits.float(), -1).gather(1, actions[:, None])[:, 0]


def _rollout(act_fn, env):
    obs, done, total = env.reset(), False, 0.0
    obs_h, act_h, rew = [], [], []
    while not done:
        a = act_fn(obs)
        nxt, r, done = env.step(a)
        obs_h.append(obs); act_h.append(a); rew.append(r); total += r
        obs = nxt
    return obs_h, act_h, rew, total


class Reinforce:
    """Monte-Carlo policy gradient with a moving-average baseline (0.9 / 0.1), gamma 0.99 (src/rl.rs:86-164)."""

    def __init__(self, obs_dim: int, n_actions: int, hidden_dim: int):
        self.policy = _policy(obs_dim, hidden_dim, n_actions, nn.Tanh)
        self.gamma, self.baseline = 0.99, 0.0

    def act(self, obs) -> int:
        with torch.no_grad():
            return sample_categorical(self.policy(_obs([obs], self.policy.device))[0].tolist())

    def train_episode(self, optimizer, env) -> float:
        obs_h, act_h, rew, total = _rollout(self.act, env)
        ret = discounted_returns(rew, self.gamma)
        optimizer.zero_grad()
        self.baseline = 0.9 * self.baseline + 0.1 * (sum(ret) / max(len(ret), 1))
        dev = self.policy.device
        logits = self.policy(_obs(obs_h, dev))
        adv = torch.tensor(ret, device=dev) - self.baseline
        loss = (-_logp(logits, torch.tensor(act_h, device=dev)) * adv).sum()      # sum_t CE_t * adv_t
        loss.backward()
        optimizer.step()
        return total

    def parameters(self):
        return self.policy.parameters()


class ActorCritic:
    """Advantage actor-critic, value coefficient 0.5 (src/rl.rs:166-255)."""

    def __init__(self, obs_dim: int, n_actions: int, hidden_dim: int):
        self.actor = _policy(obs_dim, hidden_dim, n_actions, nn.Tanh)
        self.critic = _policy(obs_dim, hidden_dim, 1, nn.Tanh)
        self.gamma, self.value_coeff = 0.99, 0.5

    def act(self, obs) -> int:
        with torch.no_grad():
            return sample_categorical(self.actor(_obs([obs], self.actor.device))[0].tolist())

    def parameters(self):
        return self.actor.parameters() + self.critic.parameters()

    def train_episode(self, optimizer, env) -> float:
        obs_h, act_h, rew, total = _rollout(self.act, env)
        dev = self.actor.device
        ret = torch.tensor(discounted_returns(rew, self.gamma), device=dev)
        optimizer.zero_grad()
        o = _obs(obs_h, dev)
        logits, value = self.actor(o), self.critic(o)[:, 0].float()
        adv = (ret - value).detach()
        loss = (-_logp(logits, torch.tensor(act_h, device=dev)) * adv).sum() + self.value_coeff * ((value - ret) ** 2).sum()
        loss.backward()
        optimizer.step()
        return total


@dataclasses.dataclass
class Transition:
    state: List[float]
    action: int
    reward: float
    next_state: List[float]
    done: bool


class ReplayBuffer:
    """Fixed-capacity ring buffer with uniform sampling (src/rl.rs:266-317)."""

    def __init__(self, capacity: int, seed: int = None):
        self.capacity, self.data, self.pos = capacity, [], 0
        self.rng = random.Random(seed)

    @staticmethod
    def new(capacity: int): return ReplayBuffer(capacity)
    @staticmethod
    def with_seed(capacity: int, seed: int): return ReplayBuffer(capacity, seed)

    def len(self) -> int: return len(self.data)
    def __len__(self): return len(self.data)
    def is_empty(self) -> bool: return not self.data

    def push(self, t: Transition):
        if len(self.data) < self.capacity:
            self.data.append(t)
        else:
            self.data[self.pos] = t
        self.pos = (self.pos + 1) % self.capacity

    def sample(self, batch_size: int) -> List[Transition]:
        return [self.data[self.rng.randrange(len(self.data))] for _ in range(batch_size)]


class Dqn:
    """DQN: Q-net Linear-ReLU-Linear-ReLU-Linear, target net, gamma .99, eps 1 -> .05 (x .995 per train
    step), target sync every 100 train steps (src/rl.rs:319-442)."""

    def __init__(self, obs_dim: int, n_actions: int, hidden_dim: int, seed: int = None):
        mk = lambda: nn.Sequential(nn.Linear(obs_dim, hidden_dim), nn.ReLU(), nn.Linear(hidden_dim, hidden_dim), nn.ReLU(),
                                   nn.Linear(hidden_dim, n_actions))
        self.q_net, self.target_net = mk(), mk()
        self.n_actions, self.gamma = n_actions, 0.99
        self.epsilon, self.epsilon_min, self.epsilon_decay, self.target_update_freq = 1.0, 0.05, 0.995, 100
        self.step_count = 0
        self.rng = random.Random(seed)
        self.sync_target()

    @staticmethod
    def new(obs_dim, n_actions, hidden_dim): return Dqn(obs_dim, n_actions, hidden_dim)
    @staticmethod
    def with_seed(obs_dim, n_actions, hidden_dim, seed): return Dqn(obs_dim, n_actions, hidden_dim, seed)

    def parameters(self):
        return self.q_net.parameters()

    def act(self, obs) -> int:
        if self.rng.random() < self.epsilon:
            return self.rng.randrange(self.n_actions)
        with torch.no_grad():
            return int(self.q_net(_obs([obs], self.q_net.device))[0].argmax())

    def sync_target(self):
        with torch.no_grad():
            for t, w in zip(self.target_net.parameters(), self.q_net.parameters()):
                if t.device != w.device:
                    t.data = t.data.to(w.device)
                t.copy_(w)

    def td_error(self, batch: List[Transition]) -> torch.Tensor:
        dev = self.q_net.device
        s = _obs([t.state for t in batch], dev); s2 = _obs([t.next_state for t in batch], dev)
        a = torch.tensor([t.action for t in batch], device=dev)
        r = torch.tensor([t.reward for t in batch], device=dev)
        nd = torch.tensor([0.0 if t.done else 1.0 for t in batch], device=dev)
        with torch.no_grad():
            y = r + self.gamma * nd * self.target_net(s2).float().max(-1).values
        q = self.q_net(s).float().gather(1, a[:, None])[:, 0]
        return q - y

    def train_step(self, buffer: ReplayBuffer, optimizer, batch_size: int):
        if buffer.len() < batch_size:
            return
        optimizer.zero_grad()
        (self.td_error(buffer.sample(batch_size)) ** 2).sum().backward()
        optimizer.step()
        self.step_count += 1
        self.epsilon = max(self.epsilon * self.epsilon_decay, self.epsilon_min)
        if self.step_count % self.target_update_freq == 0:
            self.sync_target()


def clipped_advantage_weight(adv: float, logp_old: float, logp_new: float, clip_eps: float) -> float:
    """The reference's PPO clip: the advantage weight is zeroed once the ratio leaves the trust region in the
    improving direction (src/rl.rs:600-613)."""
    ratio = math.exp(logp_new - logp_old)
    if adv >= 0:
        return 0.0 if ratio > 1 + clip_eps else adv
    return 0.0 if ratio < 1 - clip_eps else adv


class Ppo:
    """PPO with the reference's weight-zeroing clip, clip .2, value coeff .5, 4 epochs (src/rl.rs:444-598)."""

    def __init__(self, obs_dim: int, n_actions: int, hidden_dim: int):
        self.actor = _policy(obs_dim, hidden_dim, n_actions, nn.Tanh)
        self.critic = _policy(obs_dim, hidden_dim, 1, nn.Tanh)
        self.gamma, self.clip_eps, self.value_coeff, self.epochs = 0.99, 0.2, 0.5, 4

    def parameters(self):
        return self.actor.parameters() + self.critic.parameters()

    def act(self, obs) -> Tuple[int, float]:
        with torch.no_grad():
            logits = self.actor(_obs([obs], self.actor.device))[0].float()
        a = sample_categorical(logits.tolist())
        return a, float(torch.log_softmax(logits, -1)[a])

    def update(self, env, n_steps: int, optimizer) -> float:
        dev = self.actor.device
        obs, rewards, episodes = env.reset(), 0.0, 0
        t_obs, t_act, t_rew, t_val, t_logp = [], [], [], [], []
        for _ in range(n_steps):
            a, lp = self.act(obs)
            with torch.no_grad():
                v = float(self.critic(_obs([obs], dev))[0, 0])
            nxt, r, done = env.step(a)
            rewards += r
            t_obs.append(obs); t_act.append(a); t_rew.append(r); t_val.append(v); t_logp.append(lp)
            obs = nxt
            if done:
                obs = env.reset(); episodes += 1
        ret = torch.tensor(discounted_returns(t_rew, self.gamma), device=dev)
        adv = ret - torch.tensor(t_val, device=dev)
        o = _obs(t_obs, dev); acts = torch.tensor(t_act, device=dev); lp_old = torch.tensor(t_logp, device=dev)
        for _ in range(self.epochs):
            optimizer.zero_grad()
            logits, value = self.actor(o), self.critic(o)[:, 0].float()
            lp_new = _logp(logits, acts)
            ratio = torch.exp(lp_new.detach() - lp_old)
            keep = torch.where(adv >= 0, ratio <= 1 + self.clip_eps, ratio >= 1 - self.clip_eps)
            w = adv * keep.float()
            loss = (-lp_new * w).sum() + self.value_coeff * ((value - ret) ** 2).sum()
            loss.backward()
            optimizer.step()
        return rewards / episodes if episodes else rewards


class BanditEnv(Environment):
    """k-armed bandit, arm i pays with probability 0.1 + 0.8 (k-1-i)/(k-1); `deterministic` pays the probability
    itself; `sparse` pays 1 for arm 0 only (src/rl.rs:639-725). One-step episodes, observation [1.0]."""

    def __init__(self, k: int, seed: int = None, deterministic: bool = False, probs: List[float] = None):
        self.probs = probs if probs is not None else [0.1 + 0.8 * (k - 1 - i) / (k - 1) if k > 1 else 0.9 for i in range(k)]
        self.deterministic = deterministic
        self.rng = random.Random(seed)

    @staticmethod
    def new(k): return BanditEnv(k)
    @staticmethod
    def with_seed(k, seed): return BanditEnv(k, seed)
    @staticmethod
    def make_deterministic(k): return BanditEnv(k, deterministic=True)
    @staticmethod
    def deterministic(k): return BanditEnv(k, deterministic=True)      # the reference's name (src/rl.rs); instances carry the flag under the same name
    @staticmethod
    def sparse(k): return BanditEnv(k, deterministic=True, probs=[1.0] + [0.0] * (k - 1) if k > 0 else [])

    def reset(self): return [1.0]

    def step(self, action):
        p = self.probs[action]
        r = p if self.deterministic else (1.0 if self.rng.random() < p else 0.0)
        return [1.0], r, True

    def observation_dim(self): return 1
    def num_actions(self): return len(self.probs)


class ChainEnv(Environment):
    """Chain of n states, start at n-1, action 0 moves left, anything else right; reaching state 0 pays 1 and ends,
    every other step costs 0.1; at most 4n steps (src/rl.rs:727-790). One-hot observations."""

    def __init__(self, n: int, max_steps: int = None):
        self.n, self.state, self.max_steps, self.step_penalty, self.step_count = n, n - 1, max_steps or n * 4, -0.1, 0

    @staticmethod
    def new(n): return ChainEnv(n)
    @staticmethod
    def with_max_steps(n, max_steps): return ChainEnv(n, max_steps)

    def _obs(self):
        v = [0.0] * self.n; v[self.state] = 1.0
        return v

    def reset(self):
        self.state, self.step_count = self.n - 1, 0
        return self._obs()

    def step(self, action):
        if action == 0:
            self.state = max(self.state - 1, 0)
        else:
            self.state = min(self.state + 1, self.n - 1)
        self.step_count += 1
        if self.state == 0:
            return self._obs(), 1.0, True
        return self._obs(), self.step_penalty, self.step_count >= self.max_steps

    def observation_dim(self): return self.n
    def num_actions(self): return 2


from ._compat import install as _install  # noqa: E402

_install(globals())
