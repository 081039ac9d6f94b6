"""Environments: a small space/Env protocol, GridWorld and CartPole.

The reference builds on Gymnasium (rl/common/grid_world.py:33, rl/deep/cli.py:179-180), which
is not available offline; the two environments it uses are implemented here directly with the
same `reset() -> (obs, info)` / `step(a) -> (obs, reward, terminated, truncated, info)` contract.

GridWorld (rl/common/grid_world.py): N x N grid, actions up/right/down/left clipped at the
walls, step reward -0.05, goal +1 (terminal), trap -1 (terminal), truncation after 4 N^2 steps,
traps drawn from a seeded shuffle so that a start->goal path always remains (N^2 / 16 traps).
CartPole: the classic cart-pole balancing task with the CartPole-v1 constants (force 10 N,
tau 0.02 s, failure beyond 12 degrees or 2.4 m, reward 1 per step, truncation at 500 steps).
"""
from __future__ import annotations

import math
from collections import deque
from random import Random
from typing import Any

import numpy as np

Position = tuple[int, int]
ACTION_TO_DELTA: dict[int, Position] = {0: (-1, 0), 1: (0, 1), 2: (1, 0), 3: (0, -1)}
ACTION_ARROWS = {0: "^", 1: ">", 2: "v", 3: "<"}
STEP_REWARD, GOAL_REWARD, TRAP_REWARD = -0.05, 1.0, -1.0
TRAP_CELL_RATIO = 16


class Discrete:
    def __init__(self, n: int, seed: int | None = None):
        self.n = int(n)
        self._rng = np.random.default_rng(seed)

    def contains(self, x) -> bool:
        return isinstance(x, (int, np.integer)) and 0 <= int(x) < self.n

    def sample(self) -> int:
        return int(self._rng.integers(self.n))

    def seed(self, seed: int) -> None:
        self._rng = np.random.default_rng(seed)


class Box:
    def __init__(self, low, high, shape):
        self.low, self.high, self.shape = low, high, tuple(shape)


# --------------------------------------------------------------------------- grid mechanics
def encode_position(size: int, position: Position) -> int:
    return position[0] * size + position[1]


def decode_position(size: int, observation: int) -> Position:
    return divmod(int(observation), size)


def next_position(size: int, position: Position, action: int) -> Position:
    if action not in ACTION_TO_DELTA:
        raise ValueError(f"invalid action: {action}")
    dr, dc = ACTION_TO_DELTA[action]
    return (min(max(position[0] + dr, 0), size - 1), min(max(position[1] + dc, 0), size - 1))


def grid_transition(size, goal, traps, position, action) -> tuple[Position, float, bool]:
    new = next_position(size, position, action)
    if new == goal:
        return new, GOAL_REWARD, True
    if new in traps:
        return new, TRAP_REWARD, True
    return new, STEP_REWARD, False


def neighbors(size: int, position: Position) -> list[Position]:
    out = []
    for dr, dc in ACTION_TO_DELTA.values():
        r, c = position[0] + dr, position[1] + dc
        if 0 <= r < size and 0 <= c < size:
            out.append((r, c))
    return out


def has_path(size: int, start: Position, goal: Position, traps: set[Position]) -> bool:
    queue, seen = deque([start]), {start}
    while queue:
        p = queue.popleft()
        if p == goal:
            return True
        for q in neighbors(size, p):
            if q not in seen and q not in traps:
                seen.add(q)
                queue.append(q)
    return False


class GridWorldEnv:
    def __init__(self, size: int = 8, start: Position = (0, 0), goal: Position | None = None,
                 traps: tuple[Position, ...] = (), max_steps: int | None = None):
        if size < 2:
            raise ValueError("size must be at least 2")
        self.size, self.start = size, start
        self.goal = goal if goal is not None else (size - 1, size - 1)
        self.traps = set(traps)
        self.max_steps = max_steps if max_steps is not None else size * size * 4
        for name, pos in [("start", self.start), ("goal", self.goal)] + [("trap", t) for t in self.traps]:
            if not (0 <= pos[0] < size and 0 <= pos[1] < size):
                raise ValueError(f"{name} position {pos} is outside the grid")
        if self.start in self.traps or self.goal in self.traps:
            raise ValueError("start and goal cannot be traps")
        if not has_path(size, self.start, self.goal, self.traps):
            raise ValueError("traps must leave a path from start to goal")
        self.observation_space = Discrete(size * size)
        self.action_space = Discrete(4)
        self.agent_position = self.start
        self.steps = 0

    def reset(self, *, seed: int | None = None, options: dict | None = None):
        if seed is not None:
            self.action_space.seed(seed)
        self.agent_position, self.steps = self.start, 0
        return self.encode(self.agent_position), self._info()

    def step(self, action: int):
        if not self.action_space.contains(action):
            raise ValueError(f"invalid action: {action}")
        self.steps += 1
        pos, reward, terminated = grid_transition(self.size, self.goal, self.traps, self.agent_position,
                                                  int(action))
        self.agent_position = pos
        truncated = self.steps >= self.max_steps and not terminated
        return self.encode(pos), reward, terminated, truncated, self._info()

    @staticmethod
    def generate_traps(size: int, seed: int, start: Position, goal: Position) -> tuple[Position, ...]:
        target = size * size // TRAP_CELL_RATIO
        cells = [(r, c) for r in range(size) for c in range(size) if (r, c) not in {start, goal}]
        Random(seed).shuffle(cells)
        traps: set[Position] = set()
        for cell in cells:
            if len(traps) >= target:
                break
            if has_path(size, start, goal, traps | {cell}):
                traps.add(cell)
        return tuple(sorted(traps))

    def render(self) -> str:
        rows = []
        for r in range(self.size):
            row = []
            for c in range(self.size):
                p = (r, c)
                row.append("A" if p == self.agent_position else "S" if p == self.start else
                           "G" if p == self.goal else "X" if p in self.traps else ".")
            rows.append(" ".join(row))
        return "\n".join(rows)

    def render_policy(self, q_values: np.ndarray) -> str:
        rows = []
        for r in range(self.size):
            row = []
            for c in range(self.size):
                p = (r, c)
                if p == self.goal:
                    row.append("G")
                elif p == self.start:
                    row.append("S")
                elif p in self.traps:
                    row.append("X")
                else:
                    row.append(ACTION_ARROWS[int(np.argmax(q_values[self.encode(p)]))])
            rows.append(" ".join(row))
        return "\n".join(rows)

    def encode(self, position: Position) -> int:
        return encode_position(self.size, position)

    def _info(self) -> dict[str, Any]:
        p = self.agent_position
        return {"position": p, "steps": self.steps,
                "distance_to_goal": abs(p[0] - self.goal[0]) + abs(p[1] - self.goal[1]),
                "is_success": p == self.goal}


class CartPoleEnv:
    """Cart-pole balancing with the CartPole-v1 constants (Euler integration)."""

    gravity, masscart, masspole, length = 9.8, 1.0, 0.1, 0.5
    force_mag, tau = 10.0, 0.02
    theta_threshold = 12 * 2 * math.pi / 360
    x_threshold = 2.4

    def __init__(self, max_steps: int = 500):
        self.max_steps = max_steps
        self.observation_space = Box(-np.inf, np.inf, (4,))
        self.action_space = Discrete(2)
        self._rng = np.random.default_rng()
        self.state = np.zeros(4, dtype=np.float64)
        self.steps = 0

    def reset(self, *, seed: int | None = None, options: dict | None = None):
        if seed is not None:
            self._rng = np.random.default_rng(seed)
        self.state = self._rng.uniform(-0.05, 0.05, size=4)
        self.steps = 0
        return self.state.astype(np.float32), {}

    def step(self, action: int):
        x, x_dot, theta, theta_dot = self.state
        force = self.force_mag if int(action) == 1 else -self.force_mag
        total_mass = self.masspole + self.masscart
        pml = self.masspole * self.length
        cos_t, sin_t = math.cos(theta), math.sin(theta)
        temp = (force + pml * theta_dot ** 2 * sin_t) / total_mass
        theta_acc = (self.gravity * sin_t - cos_t * temp) / (
            self.length * (4.0 / 3.0 - self.masspole * cos_t ** 2 / total_mass))
        x_acc = temp - pml * theta_acc * cos_t / total_mass
        x, x_dot = x + self.tau * x_dot, x_dot + self.tau * x_acc
        theta, theta_dot = theta + self.tau * theta_dot, theta_dot + self.tau * theta_acc
        self.state = np.array([x, x_dot, theta, theta_dot])
        self.steps += 1
        terminated = bool(abs(x) > self.x_threshold or abs(theta) > self.theta_threshold)
        truncated = self.steps >= self.max_steps and not terminated
        return self.state.astype(np.float32), 1.0, terminated, truncated, {}
