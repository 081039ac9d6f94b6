"""Tabular agents on GridWorld: Monte-Carlo (sample-average and constant-alpha), TD(0) state
values under a random policy, SARSA, Expected SARSA, Q-learning, Dyna-Q.

Update rules follow rl/tabular/agents/*.py of the reference, including its treatment of episode
ends: TD-style targets bootstrap across a truncation but not across a termination; SARSA
closes the episode's last transition without a next action; the Monte-Carlo agents bootstrap
the final step of a truncated episode from max_a Q(s', a).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .core import epsilon_for_episode


@dataclass(frozen=True)
class TabularConfig:
    gamma: float = 0.99
    alpha: float = 0.1
    epsilon_start: float = 1.0
    epsilon_end: float = 0.04
    epsilon_decay_episodes: int = 200
    seed: int = 0


def greedy_action(q: np.ndarray, rng: np.random.Generator) -> int:
    """Arg-max with random tie-breaking."""
    best = np.flatnonzero(np.isclose(q, np.max(q)))
    return int(rng.choice(best))


def epsilon_greedy_action(q: np.ndarray, epsilon: float, rng: np.random.Generator) -> int:
    if rng.random() < epsilon:
        return int(rng.integers(len(q)))
    return greedy_action(q, rng)


def epsilon_greedy_probs(q: np.ndarray, epsilon: float) -> np.ndarray:
    probs = np.full(len(q), epsilon / len(q), dtype=np.float64)
    best = np.flatnonzero(np.isclose(q, np.max(q)))
    probs[best] += (1.0 - epsilon) / len(best)
    return probs


class ActionValueAgent:
    name = "tabular-action-value"

    def __init__(self, env, config: TabularConfig = TabularConfig()):
        self.config = config
        self.observation_count = int(env.observation_space.n)
        self.action_count = int(env.action_space.n)
        self.q_values = np.zeros((self.observation_count, self.action_count), dtype=np.float64)
        self.rng = np.random.default_rng(config.seed)
        self.epsilon = config.epsilon_start

    def start_episode(self, episode: int) -> None:
        self.epsilon = epsilon_for_episode(self.config, episode)

    def select_action(self, observation: int, training: bool = True) -> int:
        if training:
            return epsilon_greedy_action(self.q_values[observation], self.epsilon, self.rng)
        return greedy_action(self.q_values[observation], self.rng)

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        raise NotImplementedError

    def end_episode(self) -> None:
        pass

    def _td(self, s, a, target) -> None:
        self.q_values[s, a] += self.config.alpha * (target - self.q_values[s, a])


class TDZeroAgent:
    """TD(0) evaluation of the uniformly random policy (state values only)."""
    name = "td-zero"

    def __init__(self, env, config: TabularConfig = TabularConfig()):
        self.config = config
        self.action_count = int(env.action_space.n)
        self.v_values = np.zeros(int(env.observation_space.n), dtype=np.float64)
        self.rng = np.random.default_rng(config.seed)

    def start_episode(self, episode: int) -> None:
        pass

    def select_action(self, observation: int, training: bool = True) -> int:
        return int(self.rng.integers(self.action_count))

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        target = reward if terminated else reward + self.config.gamma * self.v_values[next_observation]
        self.v_values[observation] += self.config.alpha * (target - self.v_values[observation])

    def end_episode(self) -> None:
        pass


class _MonteCarloAgent(ActionValueAgent):
    def __init__(self, env, config: TabularConfig = TabularConfig(), first_visit: bool = True):
        super().__init__(env, config)
        self.first_visit = first_visit
        self.episode: list[tuple[int, int, float, int, bool]] = []

    def start_episode(self, episode: int) -> None:
        super().start_episode(episode)
        self.episode = []

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self.episode.append((observation, action, reward, next_observation, truncated))

    def _apply(self, s: int, a: int, ret: float) -> None:
        raise NotImplementedError

    def end_episode(self) -> None:
        g = 0.0
        returns = [0.0] * len(self.episode)
        last = len(self.episode) - 1
        for i in range(last, -1, -1):
            _, _, reward, nxt, truncated = self.episode[i]
            if truncated and i == last:
                g = reward + self.config.gamma * float(np.max(self.q_values[nxt]))
            else:
                g = reward + self.config.gamma * g
            returns[i] = g
        seen: set[tuple[int, int]] = set()
        for (s, a, _, _, _), ret in zip(self.episode, returns):
            if self.first_visit and (s, a) in seen:
                continue
            seen.add((s, a))
            self._apply(s, a, ret)


class MonteCarloAverageAgent(_MonteCarloAgent):
    name = "mc-average"

    def __init__(self, env, config: TabularConfig = TabularConfig(), first_visit: bool = True):
        super().__init__(env, config, first_visit)
        self.visit_counts = np.zeros_like(self.q_values)

    def _apply(self, s, a, ret) -> None:
        self.visit_counts[s, a] += 1.0
        self.q_values[s, a] += (ret - self.q_values[s, a]) / self.visit_counts[s, a]


class MonteCarloAlphaAgent(_MonteCarloAgent):
    name = "mc-alpha"

    def _apply(self, s, a, ret) -> None:
        self._td(s, a, ret)


class SarsaAgent(ActionValueAgent):
    name = "sarsa"

    def __init__(self, env, config: TabularConfig = TabularConfig()):
        super().__init__(env, config)
        self.pending: tuple[int, int, float, int] | None = None

    def start_episode(self, episode: int) -> None:
        super().start_episode(episode)
        self.pending = None

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        if self.pending is not None:  # this action is A_{t+1} of the previous transition
            s, a, r, s2 = self.pending
            self._td(s, a, r + self.config.gamma * self.q_values[s2, action])
        if terminated or truncated:  # no next action will ever come
            self._td(observation, action, reward)
            self.pending = None
        else:
            self.pending = (observation, action, reward, next_observation)

    def end_episode(self) -> None:
        self.pending = None


class SarsaExpectedAgent(ActionValueAgent):
    name = "sarsa-expected"

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        target = reward
        if not terminated:
            q = self.q_values[next_observation]
            target += self.config.gamma * float(np.dot(epsilon_greedy_probs(q, self.epsilon), q))
        self._td(observation, action, target)


class QLearningAgent(ActionValueAgent):
    name = "q-learning"

    def _q_update(self, s, a, r, s2, terminated) -> None:
        target = r if terminated else r + self.config.gamma * float(np.max(self.q_values[s2]))
        self._td(s, a, target)

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self._q_update(observation, action, reward, next_observation, terminated)


class DynaQAgent(QLearningAgent):
    name = "dyna-q"

    def __init__(self, env, config: TabularConfig = TabularConfig(), planning_steps: int = 8):
        super().__init__(env, config)
        self.planning_steps = planning_steps
        self.model: dict[tuple[int, int], tuple[int, float, bool]] = {}
        self.visited_keys: list[tuple[int, int]] = []

    def update(self, observation, action, reward, next_observation, terminated, truncated) -> None:
        self._q_update(observation, action, reward, next_observation, terminated)
        key = (observation, action)
        if key not in self.model:
            self.visited_keys.append(key)
        self.model[key] = (next_observation, reward, terminated)
        for _ in range(self.planning_steps):
            s, a = self.visited_keys[int(self.rng.integers(len(self.visited_keys)))]
            s2, r, term = self.model[(s, a)]
            self._q_update(s, a, r, s2, term)


AGENTS = {cls.name: cls for cls in (MonteCarloAverageAgent, MonteCarloAlphaAgent, TDZeroAgent, SarsaAgent,
                                    SarsaExpectedAgent, QLearningAgent, DynaQAgent)}
AGENT_NAMES = tuple(AGENTS)
