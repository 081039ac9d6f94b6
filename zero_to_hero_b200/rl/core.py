"""Shared RL plumbing: episode statistics, seeding, epsilon schedule, runners.

Counterparts of rl/common/type.py, seed.py, epsilon.py, grid_runner.py and rl/deep/runner.py of
the reference. An agent is anything with `start_episode(episode)`, `select_action(obs,
training)`, `update(obs, action, reward, next_obs, terminated, truncated)` and `end_episode()`.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class EpisodeStats:
    episode: int
    episode_return: float
    length: int
    terminated: bool
    truncated: bool
    is_success: bool


@dataclass(frozen=True)
class RunResult:
    agent_name: str
    episodes: list[EpisodeStats]

    def returns(self) -> np.ndarray:
        return np.array([e.episode_return for e in self.episodes], dtype=np.float64)

    def _mean(self, attr: str) -> float:
        return float(np.mean([getattr(e, attr) for e in self.episodes])) if self.episodes else 0.0

    def mean_return(self) -> float:
        return self._mean("episode_return")

    def mean_length(self) -> float:
        return sum(e.length for e in self.episodes) / max(1, len(self.episodes))

    def termination_rate(self) -> float:
        return self._mean("terminated")

    def truncation_rate(self) -> float:
        return self._mean("truncated")

    def success_rate(self) -> float:
        return self._mean("is_success")


def spawn_seeds(master_seed: int, runs: int) -> list[tuple[int, int]]:
    """(env_seed, agent_seed) per run from two independent SeedSequence children."""
    if runs < 1:
        raise ValueError("runs must be at least 1")
    env = np.random.SeedSequence(master_seed, spawn_key=(0,)).generate_state(runs)
    agent = np.random.SeedSequence(master_seed, spawn_key=(1,)).generate_state(runs)
    return [(int(e), int(a)) for e, a in zip(env, agent)]


def epsilon_for_episode(config, episode: int) -> float:
    """Linear interpolation from epsilon_start to epsilon_end over epsilon_decay_episodes."""
    progress = min(episode / max(1, config.epsilon_decay_episodes), 1.0)
    return config.epsilon_start + progress * (config.epsilon_end - config.epsilon_start)


def _grid_episode(env, agent, episode: int, training: bool) -> EpisodeStats:
    obs, info = env.reset()
    agent.start_episode(episode)
    ret, success = 0.0, False
    while True:
        action = agent.select_action(obs, training=training)
        nxt, reward, terminated, truncated, info = env.step(action)
        if training:
            agent.update(obs, action, float(reward), nxt, terminated, truncated)
        ret += float(reward)
        success = success or bool(info.get("is_success", False))
        obs = nxt
        if terminated or truncated:
            break
    agent.end_episode()
    return EpisodeStats(episode, ret, info["steps"], terminated, truncated, success)


def train_grid(env, agent, episodes: int) -> RunResult:
    return RunResult(agent.name, [_grid_episode(env, agent, e, True) for e in range(episodes)])


def evaluate_grid(env, agent, episodes: int) -> RunResult:
    return RunResult(agent.name, [_grid_episode(env, agent, e, False) for e in range(episodes)])


def _control_episode(env, agent, episode: int, seed: int, training: bool) -> EpisodeStats:
    # the environment is re-seeded per episode with seed + episode; success means the episode
    # reached the step limit (rl/deep/runner.py:49-50,83)
    obs, _ = env.reset(seed=seed + episode)
    env.action_space.seed(seed + episode)
    obs = np.asarray(obs, dtype=np.float32)
    agent.start_episode(episode)
    ret, length = 0.0, 0
    while True:
        action = agent.select_action(obs, training=training)
        nxt, reward, terminated, truncated, _ = env.step(action)
        nxt = np.asarray(nxt, dtype=np.float32)
        if training:
            agent.update(obs, action, float(reward), nxt, terminated, truncated)
        ret += float(reward)
        length += 1
        obs = nxt
        if terminated or truncated:
            break
    agent.end_episode()
    return EpisodeStats(episode, ret, length, terminated, truncated, is_success=truncated)


def train_control(env, agent, episodes: int, seed: int) -> RunResult:
    return RunResult(agent.name, [_control_episode(env, agent, e, seed, True) for e in range(episodes)])


def evaluate_control(env, agent, episodes: int, seed: int) -> RunResult:
    return RunResult(agent.name, [_control_episode(env, agent, e, seed, False) for e in range(episodes)])
