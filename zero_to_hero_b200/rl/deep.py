"""Deep RL agents for CartPole (CPU PyTorch): REINFORCE with a mean baseline, Double DQN with a
soft-updated target network, per-episode PPO with GAE and a clipped ratio, discrete Soft
Actor-Critic with twin critics.

Hyper-parameters and update rules follow rl/deep/agents/{reinforce,dqn,ppo,sac}.py of the
reference; the replay buffer here stores transitions in preallocated arrays instead of a deque
of objects, so sampling a batch is a fancy-index rather than a Python loop.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn
from torch.distributions import Categorical

from .core import epsilon_for_episode


@dataclass(frozen=True)
class DeepConfig:
    gamma: float = 0.99
    lr: float = 3e-4
    seed: int = 24
    hidden_size: int = 128
    debug: bool = False
    batch_size: int = 128
    replay_size: int = 1024 * 16
    warmup_steps: int = 1024 * 2


@dataclass(frozen=True)
class Transition:
    observation: np.ndarray
    action: int
    reward: float
    next_observation: np.ndarray
    terminated: bool
    truncated: bool


class MLP(nn.Module):
    def __init__(self, input_size: int, hidden_size: int, output_size: int):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(input_size, hidden_size), nn.ReLU(),
                                 nn.Linear(hidden_size, hidden_size), nn.ReLU(),
                                 nn.Linear(hidden_size, output_size))

    def forward(self, x):
        return self.net(x)


class ReplayBuffer:
    """Ring buffer; `sample` draws without replacement."""

    def __init__(self, capacity: int, seed: int, observation_size: int = 4):
        self.capacity, self.size, self.pos = capacity, 0, 0
        self.obs = np.zeros((capacity, observation_size), dtype=np.float32)
        self.next_obs = np.zeros((capacity, observation_size), dtype=np.float32)
        self.actions = np.zeros(capacity, dtype=np.int64)
        self.rewards = np.zeros(capacity, dtype=np.float32)
        self.terminated = np.zeros(capacity, dtype=np.float32)
        self.rng = np.random.default_rng(seed)

    def __len__(self) -> int:
        return self.size

    def append(self, t: Transition) -> None:
        i = self.pos
        self.obs[i], self.next_obs[i] = t.observation, t.next_observation
        self.actions[i], self.rewards[i], self.terminated[i] = t.action, t.reward, float(t.terminated)
        self.pos = (self.pos + 1) % self.capacity
        self.size = min(self.size + 1, self.capacity)

    def sample(self, batch_size: int):
        idx = self.rng.choice(self.size, size=batch_size, replace=False)
        return (torch.from_numpy(self.obs[idx]), torch.from_numpy(self.actions[idx]),
                torch.from_numpy(self.rewards[idx]), torch.from_numpy(self.next_obs[idx]),
                torch.from_numpy(self.terminated[idx]))


def env_sizes(env) -> tuple[int, int]:
    return int(np.prod(env.observation_space.shape)), int(env.action_space.n)


def _t(obs) -> torch.Tensor:
    return torch.as_tensor(obs, dtype=torch.float32)


class ReinforceAgent:
    name = "reinforce"

    def __init__(self, env, config: DeepConfig = DeepConfig()):
        torch.manual_seed(config.seed)
        self.config = config
        n_obs, n_act = env_sizes(env)
        self.policy = MLP(n_obs, config.hidden_size, n_act)
        self.optimizer = torch.optim.Adam(self.policy.parameters(), lr=config.lr)
        self.log_probs: list[torch.Tensor] = []
        self.rewards: list[float] = []

    def start_episode(self, episode: int) -> None:
        self.log_probs, self.rewards = [], []

    def select_action(self, observation, training: bool = True) -> int:
        logits = self.policy(_t(observation))
        if not training:
            return int(torch.argmax(logits.detach()).item())
        dist = Categorical(logits=logits)
        action = dist.sample()
        self.log_probs.append(dist.log_prob(action))
        return int(action.item())

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self.rewards.append(reward)

    def end_episode(self) -> None:
        if not self.rewards:
            return
        g, returns = 0.0, []
        for r in reversed(self.rewards):
            g = r + self.config.gamma * g
            returns.append(g)
        returns.reverse()
        ret = torch.as_tensor(returns, dtype=torch.float32)
        ret = ret - ret.mean()
        loss = -(torch.stack(self.log_probs) * ret).mean()
        self.optimizer.zero_grad()
        loss.backward()
        self.optimizer.step()


@dataclass(frozen=True)
class DQNConfig:
    epsilon_start: float = 1.0
    epsilon_end: float = 0.05
    epsilon_decay_episodes: int = 256
    target_tau: float = 0.005
    gradient_clip: float = 1


def _soft_update(target: nn.Module, online: nn.Module, tau: float) -> None:
    with torch.no_grad():
        for tp, p in zip(target.parameters(), online.parameters()):
            tp.lerp_(p, tau)


class DQNAgent:
    name = "dqn"

    def __init__(self, env, config: DeepConfig = DeepConfig(), dqn: DQNConfig = DQNConfig()):
        torch.manual_seed(config.seed)
        self.rng = np.random.default_rng(config.seed)
        self.config, self.dqn = config, dqn
        n_obs, self.action_count = env_sizes(env)
        self.q = MLP(n_obs, config.hidden_size, self.action_count)
        self.target_q = MLP(n_obs, config.hidden_size, self.action_count)
        self.target_q.load_state_dict(self.q.state_dict())
        self.optimizer = torch.optim.AdamW(self.q.parameters(), lr=config.lr, amsgrad=True)
        self.replay = ReplayBuffer(config.replay_size, config.seed, n_obs)
        self.steps, self.episode, self.epsilon = 0, 0, dqn.epsilon_start

    def start_episode(self, episode: int) -> None:
        self.episode = episode
        self.epsilon = epsilon_for_episode(self.dqn, episode)

    def select_action(self, observation, training: bool = True) -> int:
        if training and self.rng.random() < self.epsilon:
            return int(self.rng.integers(self.action_count))
        with torch.no_grad():
            return int(torch.argmax(self.q(_t(observation))).item())

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self.replay.append(Transition(observation, action, reward, next_observation, terminated, truncated))
        self.steps += 1
        if len(self.replay) < max(self.config.warmup_steps, self.config.batch_size):
            return
        obs, actions, rewards, nxt, term = self.replay.sample(self.config.batch_size)
        q = self.q(obs).gather(1, actions.unsqueeze(1)).squeeze(1)
        with torch.no_grad():
            best = self.q(nxt).argmax(dim=1)  # Double DQN: online net picks, target net rates
            next_q = self.target_q(nxt).gather(1, best.unsqueeze(1)).squeeze(1)
            targets = rewards + self.config.gamma * (1.0 - term) * next_q
        loss = nn.functional.smooth_l1_loss(q, targets)
        self.optimizer.zero_grad()
        loss.backward()
        nn.utils.clip_grad_value_(self.q.parameters(), self.dqn.gradient_clip)
        self.optimizer.step()
        _soft_update(self.target_q, self.q, self.dqn.target_tau)
        if self.config.debug and self.steps % 1000 == 0:
            print(f"episode={self.episode} step={self.steps} q: {summary(q)} target: {summary(targets)} "
                  f"gradients: {gradient_summary(self.q)}")

    def end_episode(self) -> None:
        pass


def summary(values: torch.Tensor) -> str:
    v = values.detach()
    return f"mean={v.mean().item():.2f} p95={v.quantile(0.95).item():.2f} max={v.max().item():.2f}"


def gradient_summary(module: nn.Module) -> str:
    grads = [p.grad.abs().max().item() for p in module.parameters() if p.grad is not None]
    return f"max_abs={max(grads):.4f}" if grads else "none"


@dataclass(frozen=True)
class PPOConfig:
    epochs: int = 4
    clip_ratio: float = 0.2
    gae_lambda: float = 0.95
    value_coef: float = 0.5
    entropy_coef: float = 0.01
    gradient_clip: float = 0.5


@dataclass(frozen=True)
class RolloutStep:
    transition: Transition
    log_prob: torch.Tensor
    value: torch.Tensor


class PPOAgent:
    name = "ppo"

    def __init__(self, env, config: DeepConfig = DeepConfig(), ppo: PPOConfig = PPOConfig()):
        torch.manual_seed(config.seed)
        self.config, self.ppo = config, ppo
        n_obs, n_act = env_sizes(env)
        self.policy = MLP(n_obs, config.hidden_size, n_act)
        self.value = MLP(n_obs, config.hidden_size, 1)
        self.parameters = list(self.policy.parameters()) + list(self.value.parameters())
        self.optimizer = torch.optim.Adam(self.parameters, lr=config.lr)
        self.rollout: list[RolloutStep] = []
        self.pending_step: tuple[torch.Tensor, torch.Tensor] | None = None

    def start_episode(self, episode: int) -> None:
        self.rollout, self.pending_step = [], None

    @torch.no_grad()
    def select_action(self, observation, training: bool = True) -> int:
        obs = _t(observation)
        logits = self.policy(obs)
        if not training:
            return int(torch.argmax(logits).item())
        dist = Categorical(logits=logits)
        action = dist.sample()
        self.pending_step = (dist.log_prob(action), self.value(obs).squeeze())
        return int(action.item())

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        if self.pending_step is None:
            return
        log_prob, value = self.pending_step
        self.rollout.append(RolloutStep(
            Transition(observation, action, reward, next_observation, terminated, truncated), log_prob, value))
        self.pending_step = None

    def end_episode(self) -> None:
        if self.rollout:
            self._update()

    def _advantages(self, values: torch.Tensor) -> torch.Tensor:
        """GAE over the stored episode. As in the reference, the "next value" of a step is the
        stored value of the step after it and is zero after the last one."""
        out, adv, next_value = [], 0.0, 0.0
        for i in reversed(range(len(self.rollout))):
            tr = self.rollout[i].transition
            mask = 1.0 - float(tr.terminated or tr.truncated)
            delta = tr.reward + self.config.gamma * next_value * mask - values[i].item()
            adv = delta + self.config.gamma * self.ppo.gae_lambda * mask * adv
            out.append(adv)
            next_value = values[i].item()
        out.reverse()
        return torch.as_tensor(out, dtype=torch.float32)

    def _update(self) -> None:
        obs = torch.as_tensor(np.array([s.transition.observation for s in self.rollout]), dtype=torch.float32)
        actions = torch.as_tensor([s.transition.action for s in self.rollout], dtype=torch.int64)
        old_log_probs = torch.stack([s.log_prob for s in self.rollout])
        old_values = torch.stack([s.value for s in self.rollout])
        adv = self._advantages(old_values)
        returns = adv + old_values
        if len(adv) > 1:
            adv = (adv - adv.mean()) / (adv.std() + 1e-8)
        for _ in range(self.ppo.epochs):
            order = torch.randperm(len(actions))
            for start in range(0, len(actions), self.config.batch_size):
                idx = order[start:start + self.config.batch_size]
                dist = Categorical(logits=self.policy(obs[idx]))
                ratio = torch.exp(dist.log_prob(actions[idx]) - old_log_probs[idx])
                clipped = ratio.clamp(1.0 - self.ppo.clip_ratio, 1.0 + self.ppo.clip_ratio)
                policy_loss = -torch.minimum(ratio * adv[idx], clipped * adv[idx]).mean()
                value_loss = nn.functional.mse_loss(self.value(obs[idx]).squeeze(1), returns[idx])
                loss = policy_loss + self.ppo.value_coef * value_loss - self.ppo.entropy_coef * dist.entropy().mean()
                self.optimizer.zero_grad()
                loss.backward()
                nn.utils.clip_grad_norm_(self.parameters, self.ppo.gradient_clip)
                self.optimizer.step()


@dataclass(frozen=True)
class SACConfig:
    alpha: float = 0.2
    target_tau: float = 0.005


class SACAgent:
    name = "sac"

    def __init__(self, env, config: DeepConfig = DeepConfig(), sac: SACConfig = SACConfig()):
        torch.manual_seed(config.seed)
        self.config, self.sac = config, sac
        n_obs, n_act = env_sizes(env)
        mk = lambda: MLP(n_obs, config.hidden_size, n_act)  # noqa: E731
        self.policy, self.c1, self.c2, self.target_c1, self.target_c2 = mk(), mk(), mk(), mk(), mk()
        self.target_c1.load_state_dict(self.c1.state_dict())
        self.target_c2.load_state_dict(self.c2.state_dict())
        self.policy_optimizer = torch.optim.Adam(self.policy.parameters(), lr=config.lr)
        self.critic_optimizer = torch.optim.Adam(list(self.c1.parameters()) + list(self.c2.parameters()),
                                                 lr=config.lr)
        self.replay = ReplayBuffer(config.replay_size, config.seed, n_obs)
        self.steps = 0

    def start_episode(self, episode: int) -> None:
        pass

    def select_action(self, observation, training: bool = True) -> int:
        with torch.no_grad():
            logits = self.policy(_t(observation))
        if training:
            return int(Categorical(logits=logits).sample().item())
        return int(torch.argmax(logits).item())

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self.replay.append(Transition(observation, action, reward, next_observation, terminated, truncated))
        self.steps += 1
        if len(self.replay) < max(self.config.warmup_steps, self.config.batch_size):
            return
        obs, actions, rewards, nxt, term = self.replay.sample(self.config.batch_size)
        # critics: soft Bellman target with the expectation over the policy taken in closed form
        q1 = self.c1(obs).gather(1, actions.unsqueeze(1)).squeeze(1)
        q2 = self.c2(obs).gather(1, actions.unsqueeze(1)).squeeze(1)
        with torch.no_grad():
            logits = self.policy(nxt)
            probs, log_probs = logits.softmax(dim=1), logits.log_softmax(dim=1)
            next_q = torch.minimum(self.target_c1(nxt), self.target_c2(nxt))
            next_v = (probs * (next_q - self.sac.alpha * log_probs)).sum(dim=1)
            target = rewards + self.config.gamma * (1.0 - term) * next_v
        critic_loss = nn.functional.mse_loss(q1, target) + nn.functional.mse_loss(q2, target)
        self.critic_optimizer.zero_grad()
        critic_loss.backward()
        self.critic_optimizer.step()
        # policy: minimise E_pi[alpha log pi - Q]
        logits = self.policy(obs)
        probs, log_probs = logits.softmax(dim=1), logits.log_softmax(dim=1)
        q = torch.minimum(self.c1(obs), self.c2(obs)).detach()
        policy_loss = (probs * (self.sac.alpha * log_probs - q)).sum(dim=1).mean()
        self.policy_optimizer.zero_grad()
        policy_loss.backward()
        self.policy_optimizer.step()
        _soft_update(self.target_c1, self.c1, self.sac.target_tau)
        _soft_update(self.target_c2, self.c2, self.sac.target_tau)

    def end_episode(self) -> None:
        pass


AGENTS = {cls.name: cls for cls in (ReinforceAgent, DQNAgent, PPOAgent, SACAgent)}
AGENT_NAMES = tuple(AGENTS)
