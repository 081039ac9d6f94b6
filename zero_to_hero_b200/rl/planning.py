"""Planning agents that know GridWorld's transition function: value iteration, policy
iteration and Monte-Carlo tree search with UCT.

Counterparts of rl/planning/agents/{vi,pi,mcts}.py of the reference. MCTS keeps its
GridWorld heuristics: candidate actions are those that move (preferring ones that do not step
into a trap), rollouts follow the BFS distance-to-goal map with probability 1 - rollout_epsilon,
the final choice prefers children closer to the goal, then mean return, then visit count.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field

import numpy as np

from .envs import GridWorldEnv, Position, decode_position, encode_position, grid_transition, neighbors, next_position


@dataclass(frozen=True)
class PlanningConfig:
    gamma: float = 0.99
    alpha: float = 0.1
    seed: int = 0


class _ModelBased:
    def __init__(self, env, config: PlanningConfig):
        if not isinstance(env, GridWorldEnv):
            raise TypeError(f"{type(self).__name__} requires GridWorldEnv")
        self.config = config
        self.size, self.goal, self.traps = env.size, env.goal, set(env.traps)
        self.action_count = int(env.action_space.n)
        self.state_count = int(env.observation_space.n)
        self.terminal = {encode_position(self.size, self.goal),
                         *(encode_position(self.size, t) for t in self.traps)}

    def start_episode(self, episode: int) -> None:
        pass

    def update(self, *args, **kwargs) -> None:
        pass

    def end_episode(self) -> None:
        pass

    def _backup(self, obs: int, action: int, v: np.ndarray) -> float:
        pos, reward, terminated = grid_transition(self.size, self.goal, self.traps,
                                                  decode_position(self.size, obs), action)
        return reward if terminated else reward + self.config.gamma * v[encode_position(self.size, pos)]


class ValueIterationAgent(_ModelBased):
    name = "value-iteration"

    def __init__(self, env, config: PlanningConfig = PlanningConfig(), theta: float = 1e-6):
        super().__init__(env, config)
        v = np.zeros(self.state_count)
        policy = np.zeros(self.state_count, dtype=np.int64)
        self.sweeps = 0
        while True:
            delta = 0.0
            for s in range(self.state_count):
                if s in self.terminal:
                    continue
                values = [self._backup(s, a, v) for a in range(self.action_count)]
                best = int(np.argmax(values))  # first maximiser, as a strict > scan gives
                delta = max(delta, abs(values[best] - v[s]))
                v[s], policy[s] = values[best], best
            self.sweeps += 1
            if delta < theta:
                break
        self.v, self.policy = v, policy

    def select_action(self, observation: int, training: bool = True) -> int:
        return int(self.policy[observation])


class PolicyIterationAgent(_ModelBased):
    name = "policy-iteration"

    def __init__(self, env, config: PlanningConfig = PlanningConfig(), theta: float = 1e-6):
        super().__init__(env, config)
        v = np.zeros(self.state_count)
        policy = np.zeros(self.state_count, dtype=np.int64)
        self.improvements = 0
        while True:
            while True:  # policy evaluation
                delta = 0.0
                for s in range(self.state_count):
                    if s in self.terminal:
                        continue
                    new = self._backup(s, int(policy[s]), v)
                    delta = max(delta, abs(new - v[s]))
                    v[s] = new
                if delta < theta:
                    break
            stable = True  # policy improvement
            for s in range(self.state_count):
                if s in self.terminal:
                    continue
                values = [self._backup(s, a, v) for a in range(self.action_count)]
                best = int(np.argmax(values))
                if values[best] > values[int(policy[s])] + 1e-12:
                    policy[s] = best
                    stable = False
            self.improvements += 1
            if stable:
                break
        self.v, self.policy = v, policy

    def select_action(self, observation: int, training: bool = True) -> int:
        return int(self.policy[observation])


@dataclass(frozen=True)
class MCTSConfig:
    search_depth: int | None = None
    simulation_count: int = 16
    exploration_weight: float = math.sqrt(2.0)
    rollout_epsilon: float = 0.1


@dataclass
class _Node:
    position: Position
    depth: int
    terminal: bool = False
    visits: int = 0
    value_sum: float = 0.0
    untried: list[int] = field(default_factory=list)
    edges: dict[int, "_Edge"] = field(default_factory=dict)

    def mean_value(self) -> float:
        return self.value_sum / max(1, self.visits)


@dataclass
class _Edge:
    action: int
    reward: float
    child: _Node

    def mean_return(self, gamma: float) -> float:
        return self.reward + gamma * self.child.mean_value()


class MCTSAgent(_ModelBased):
    name = "mcts"

    def __init__(self, env, config: PlanningConfig = PlanningConfig(), mcts: MCTSConfig = MCTSConfig()):
        super().__init__(env, config)
        if mcts.simulation_count < 1:
            raise ValueError("simulation_count must be at least 1")
        if not 0.0 <= mcts.rollout_epsilon <= 1.0:
            raise ValueError("rollout_epsilon must be between 0 and 1")
        self.mcts = mcts
        self.search_depth = mcts.search_depth if mcts.search_depth is not None else env.size
        self.rng = np.random.default_rng(config.seed)
        self.goal_distances = {self.goal: 0}
        queue = deque([self.goal])
        while queue:
            p = queue.popleft()
            for q in neighbors(self.size, p):
                if q not in self.goal_distances and q not in self.traps:
                    self.goal_distances[q] = self.goal_distances[p] + 1
                    queue.append(q)

    # ---- heuristics
    def _distance(self, p: Position) -> int:
        return self.goal_distances.get(p, self.size * self.size)

    def _candidates(self, p: Position) -> list[int]:
        moving = [a for a in range(self.action_count) if next_position(self.size, p, a) != p]
        safe = [a for a in moving if next_position(self.size, p, a) not in self.traps]
        return safe or moving

    def _pick(self, items: list) -> int:
        return items[int(self.rng.integers(len(items)))]

    def _rollout_action(self, p: Position) -> int:
        if self.rng.random() < self.mcts.rollout_epsilon:
            return int(self.rng.integers(self.action_count))
        scored = [(self._distance(next_position(self.size, p, a)), a) for a in self._candidates(p)]
        if not scored:
            return int(self.rng.integers(self.action_count))
        best = min(d for d, _ in scored)
        return self._pick([a for d, a in scored if d == best])

    # ---- search
    def select_action(self, observation: int, training: bool = True) -> int:
        root = _Node(decode_position(self.size, observation), 0)
        root.untried = self._candidates(root.position)
        for _ in range(self.mcts.simulation_count):
            self._simulate(root)
        edges = list(root.edges.values())
        forward = [e for e in edges if self._distance(e.child.position) < self._distance(root.position)]
        edges = forward or edges
        g = self.config.gamma
        best_value = max(e.mean_return(g) for e in edges)
        tied = [e for e in edges if math.isclose(e.mean_return(g), best_value)]
        most = max(e.child.visits for e in tied)
        return self._pick([e.action for e in tied if e.child.visits == most])

    def _simulate(self, root: _Node) -> None:
        path: list[tuple[_Edge | None, _Node]] = [(None, root)]
        node = root
        while not node.terminal and node.depth < self.search_depth and not node.untried and node.edges:
            scores = [(self._uct(node, e), e) for e in node.edges.values()]
            top = max(s for s, _ in scores)
            edge = self._pick([e for s, e in scores if math.isclose(s, top)])
            node = edge.child
            path.append((edge, node))
        value = 0.0
        if not node.terminal and node.depth < self.search_depth:
            action = node.untried.pop(int(self.rng.integers(len(node.untried))))
            pos, reward, terminal = grid_transition(self.size, self.goal, self.traps, node.position, action)
            child = _Node(pos, node.depth + 1, terminal, untried=self._candidates(pos))
            edge = _Edge(action, reward, child)
            node.edges[action] = edge
            path.append((edge, child))
            value = self._rollout(child)
        for i in range(len(path) - 1, -1, -1):
            edge, n = path[i]
            n.visits += 1
            n.value_sum += value
            if i > 0:
                value = edge.reward + self.config.gamma * value

    def _uct(self, node: _Node, edge: _Edge) -> float:
        visits = max(1, edge.child.visits)
        return edge.mean_return(self.config.gamma) + self.mcts.exploration_weight * math.sqrt(
            math.log(max(1, node.visits)) / visits)

    def _rollout(self, node: _Node) -> float:
        value, discount = 0.0, 1.0
        pos, depth, terminal = node.position, node.depth, node.terminal
        while not terminal and depth < self.search_depth:
            pos, reward, terminal = grid_transition(self.size, self.goal, self.traps, pos,
                                                    self._rollout_action(pos))
            value += discount * reward
            discount *= self.config.gamma
            depth += 1
        return value


AGENTS = {cls.name: cls for cls in (ValueIterationAgent, PolicyIterationAgent, MCTSAgent)}
AGENT_NAMES = tuple(AGENTS)
