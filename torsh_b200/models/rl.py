"""Reinforcement-learning models: DQN (plain / dueling / double targets) with a replay buffer, PPO (actor, critic, clipped
objective, generalised advantage estimation) and an A3C-style shared actor-critic with n-step returns.
Reference: crates/torsh-models/src/rl.rs (DQNConfig / DQN, PPOConfig / PPOActor / PPOCritic / PPO, A3CConfig / A3C).
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import torch
from torch import nn


def _mlp(sizes, act=nn.ReLU, out_act=None):
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2:
            layers.append(act())
        elif out_act is not None:
            layers.append(out_act())
    return nn.Sequential(*layers)


# ---- DQN ---------------------------------------------------------------------------------------------------------
@dataclass
class DQNConfig:
    state_dim: int = 4
    action_dim: int = 2
    hidden: tuple = (128, 128)
    dueling: bool = False
    double: bool = True
    gamma: float = 0.99
    epsilon: float = 0.1


class DQN(nn.Module):
    def __init__(self, cfg: DQNConfig | None = None):
        super().__init__()
        self.cfg = cfg or DQNConfig()
        c = self.cfg
        self.body = _mlp([c.state_dim, *c.hidden], out_act=nn.ReLU)
        if c.dueling:
            self.value, self.adv = nn.Linear(c.hidden[-1], 1), nn.Linear(c.hidden[-1], c.action_dim)
        else:
            self.q = nn.Linear(c.hidden[-1], c.action_dim)

    def forward(self, state):
        h = self.body(state)
        if self.cfg.dueling:
            a = self.adv(h)
            return self.value(h) + a - a.mean(-1, keepdim=True)
        return self.q(h)

    @torch.no_grad()
    def act(self, state, epsilon: float | None = None, rng: random.Random | None = None) -> int:
        eps = self.cfg.epsilon if epsilon is None else epsilon
        if (rng or random).random() < eps:
            return (rng or random).randrange(self.cfg.action_dim)
        return int(self(state.reshape(1, -1)).argmax(-1))

    def td_loss(self, target_net: "DQN", batch) -> torch.Tensor:
        """Huber loss of Q(s, a) against r + gamma * max_a' Q_target(s', a') (action chosen by the online net when
        ``double``); ``batch`` = (states, actions, rewards, next_states, dones)."""
        s, a, r, s2, d = batch
        q = self(s).gather(1, a.long()[:, None]).squeeze(1)
        with torch.no_grad():
            if self.cfg.double:
                a2 = self(s2).argmax(-1, keepdim=True)
                q2 = target_net(s2).gather(1, a2).squeeze(1)
            else:
                q2 = target_net(s2).max(-1).values
            y = r + self.cfg.gamma * (1 - d.float()) * q2
        return nn.functional.smooth_l1_loss(q, y)


class ReplayBuffer:
    def __init__(self, capacity: int, state_dim: int, seed: int = 0):
        self.cap, self.n, self.pos = capacity, 0, 0
        self.s, self.s2 = torch.zeros(capacity, state_dim), torch.zeros(capacity, state_dim)
        self.a, self.r, self.d = torch.zeros(capacity, dtype=torch.long), torch.zeros(capacity), torch.zeros(capacity, dtype=torch.bool)
        self.gen = torch.Generator().manual_seed(seed)

    def push(self, s, a, r, s2, done):
        i = self.pos
        self.s[i], self.a[i], self.r[i], self.s2[i], self.d[i] = torch.as_tensor(s), int(a), float(r), torch.as_tensor(s2), bool(done)
        self.pos = (i + 1) % self.cap
        self.n = min(self.n + 1, self.cap)

    def __len__(self): return self.n

    def sample(self, batch_size: int):
        idx = torch.randint(0, self.n, (batch_size,), generator=self.gen)
        return self.s[idx], self.a[idx], self.r[idx], self.s2[idx], self.d[idx]


# ---- PPO ---------------------------------------------------------------------------------------------------------
@dataclass
class PPOConfig:
    state_dim: int = 4
    action_dim: int = 2
    hidden: tuple = (64, 64)
    continuous: bool = False
    clip: float = 0.2
    gamma: float = 0.99
    lam: float = 0.95
    value_coef: float = 0.5
    entropy_coef: float = 0.01


class PPOActor(nn.Module):
    def __init__(self, cfg: PPOConfig):
        super().__init__()
        self.cfg = cfg
        self.net = _mlp([cfg.state_dim, *cfg.hidden, cfg.action_dim], act=nn.Tanh)
        if cfg.continuous:
            self.log_std = nn.Parameter(torch.zeros(cfg.action_dim))

    def dist(self, state):
        out = self.net(state)
        if self.cfg.continuous:
            return torch.distributions.Independent(torch.distributions.Normal(out, self.log_std.exp()), 1)
        return torch.distributions.Categorical(logits=out)


class PPOCritic(nn.Module):
    def __init__(self, cfg: PPOConfig):
        super().__init__()
        self.net = _mlp([cfg.state_dim, *cfg.hidden, 1], act=nn.Tanh)

    def forward(self, state):
        return self.net(state).squeeze(-1)


def gae(rewards, values, dones, last_value, gamma: float = 0.99, lam: float = 0.95):
    """Generalised advantage estimates and returns for one trajectory (1-D tensors of length T)."""
    T = rewards.shape[0]
    adv = torch.zeros(T)
    running, nxt = 0.0, last_value
    for t in range(T - 1, -1, -1):
        mask = 1.0 - float(dones[t])
        delta = rewards[t] + gamma * nxt * mask - values[t]
        running = delta + gamma * lam * mask * running
        adv[t] = running
        nxt = values[t]
    return adv, adv + values


class PPO(nn.Module):
    def __init__(self, cfg: PPOConfig | None = None):
        super().__init__()
        self.cfg = cfg or PPOConfig()
        self.actor, self.critic = PPOActor(self.cfg), PPOCritic(self.cfg)

    @torch.no_grad()
    def act(self, state):
        d = self.actor.dist(state)
        a = d.sample()
        return a, d.log_prob(a), self.critic(state)

    def loss(self, states, actions, old_log_probs, advantages, returns) -> dict:
        c = self.cfg
        d = self.actor.dist(states)
        ratio = torch.exp(d.log_prob(actions) - old_log_probs)
        adv = (advantages - advantages.mean()) / (advantages.std() + 1e-8)
        policy = -torch.min(ratio * adv, ratio.clamp(1 - c.clip, 1 + c.clip) * adv).mean()
        value = nn.functional.mse_loss(self.critic(states), returns)
        entropy = d.entropy().mean()
        return {"policy": policy, "value": value, "entropy": entropy, "total": policy + c.value_coef * value - c.entropy_coef * entropy}


# ---- A3C ---------------------------------------------------------------------------------------------------------
@dataclass
class A3CConfig:
    state_dim: int = 4
    action_dim: int = 2
    hidden: int = 128
    gamma: float = 0.99
    value_coef: float = 0.5
    entropy_coef: float = 0.01


class A3C(nn.Module):
    """Shared trunk with policy and value heads; workers compute ``loss`` on n-step rollouts and apply their gradients to
    a shared copy (``share_memory()`` + one optimizer per worker is the classic arrangement)."""

    def __init__(self, cfg: A3CConfig | None = None):
        super().__init__()
        self.cfg = cfg or A3CConfig()
        c = self.cfg
        self.trunk = _mlp([c.state_dim, c.hidden, c.hidden], out_act=nn.ReLU)
        self.policy, self.value = nn.Linear(c.hidden, c.action_dim), nn.Linear(c.hidden, 1)

    def forward(self, state):
        h = self.trunk(state)
        return self.policy(h), self.value(h).squeeze(-1)

    def loss(self, states, actions, rewards, bootstrap_value: float = 0.0) -> torch.Tensor:
        c = self.cfg
        logits, values = self(states)
        R, rets = bootstrap_value, []
        for r in reversed(rewards.tolist()):
            R = r + c.gamma * R
            rets.append(R)
        rets = torch.tensor(rets[::-1])
        adv = rets - values
        logp = torch.log_softmax(logits, -1)
        chosen = logp.gather(1, actions.long()[:, None]).squeeze(1)
        entropy = -(logp.exp() * logp).sum(-1).mean()
        return -(chosen * adv.detach()).mean() + c.value_coef * adv.pow(2).mean() - c.entropy_coef * entropy
