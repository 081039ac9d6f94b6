"""RL: environment mechanics, exact TD targets (termination vs truncation), GAE numbers, and
end-to-end learning on tiny problems (CPU). Mirrors the reference's rl test suites."""
import numpy as np
import pytest
import torch

from zero_to_hero_b200.rl import deep, planning, tabular
from zero_to_hero_b200.rl.core import (evaluate_control, evaluate_grid, spawn_seeds, train_control,
                                       train_grid, epsilon_for_episode)
from zero_to_hero_b200.rl.envs import CartPoleEnv, GridWorldEnv


def test_spawn_seeds_deterministic_and_distinct():
    a, b = spawn_seeds(24, 4), spawn_seeds(24, 4)
    assert a == b and len({s for pair in a for s in pair}) == 8
    assert spawn_seeds(25, 4) != a
    with pytest.raises(ValueError):
        spawn_seeds(1, 0)


def test_gridworld_mechanics():
    env = GridWorldEnv(size=3, traps=((1, 1),))
    obs, info = env.reset()
    assert obs == 0 and info["distance_to_goal"] == 4
    obs, r, term, trunc, _ = env.step(0)  # up at the wall: stays
    assert (obs, r, term) == (0, -0.05, False)
    obs, r, term, _, _ = env.step(1)
    assert obs == 1
    obs, r, term, _, _ = env.step(2)  # into the trap
    assert (obs, r, term) == (4, -1.0, True)
    env.reset()
    for a in (1, 1, 2, 2):
        obs, r, term, _, info = env.step(a)
    assert (obs, r, term, info["is_success"]) == (8, 1.0, True, True)
    with pytest.raises(ValueError):
        GridWorldEnv(size=2, traps=((0, 1), (1, 0)))  # no path left
    t1 = GridWorldEnv.generate_traps(8, 24, (0, 0), (7, 7))
    assert t1 == GridWorldEnv.generate_traps(8, 24, (0, 0), (7, 7)) and len(t1) == 4
    small = GridWorldEnv(size=2, max_steps=3)
    small.reset()
    out = [small.step(0) for _ in range(3)]
    assert out[-1][3] is True and out[-1][2] is False  # truncated, not terminated
    assert "A" in env.render() and "G" in env.render_policy(np.zeros((9, 4)))


def test_epsilon_schedule():
    cfg = tabular.TabularConfig()
    assert epsilon_for_episode(cfg, 0) == 1.0
    assert epsilon_for_episode(cfg, 100) == pytest.approx(0.52)
    assert epsilon_for_episode(cfg, 10_000) == pytest.approx(0.04)


def _cfg():
    return tabular.TabularConfig(alpha=0.5, gamma=0.8, epsilon_start=0.0)


def test_bootstrapping_across_truncation_but_not_termination():
    env = GridWorldEnv(size=3)
    for cls in (tabular.QLearningAgent, tabular.SarsaExpectedAgent):
        agent = cls(env, _cfg())
        agent.q_values[1] = [1.0, 2.0, 0.0, -1.0]
        agent.update(0, 1, -0.1, 1, terminated=False, truncated=True)
        assert agent.q_values[0, 1] == pytest.approx(0.75)
    td = tabular.TDZeroAgent(env, _cfg())
    td.v_values[1] = 2.0
    td.update(0, 1, -0.1, 1, False, True)
    assert td.v_values[0] == pytest.approx(0.75)
    td = tabular.TDZeroAgent(env, _cfg())
    td.v_values[1] = 2.0
    td.update(0, 1, 1.0, 1, True, False)
    assert td.v_values[0] == pytest.approx(0.5)
    mc = tabular.MonteCarloAlphaAgent(env, _cfg())
    mc.q_values[1] = [1.0, 2.0, 0.0, -1.0]
    mc.update(0, 1, -0.1, 1, False, True)
    mc.end_episode()
    assert mc.q_values[0, 1] == pytest.approx(0.75)


def test_sarsa_uses_the_action_actually_taken_next():
    agent = tabular.SarsaAgent(GridWorldEnv(size=3), _cfg())
    agent.q_values[1] = [1.0, 2.0, 0.0, -1.0]
    agent.start_episode(0)
    agent.update(0, 1, -0.1, 1, False, False)
    assert agent.q_values[0, 1] == 0.0  # waits for A_{t+1}
    agent.update(1, 3, -0.1, 0, False, False)  # A_{t+1} = 3 with Q = -1
    assert agent.q_values[0, 1] == pytest.approx(0.5 * (-0.1 + 0.8 * -1.0))
    agent.update(0, 2, 1.0, 3, True, False)  # terminal: closes both pending and final transition
    assert agent.q_values[0, 2] == pytest.approx(0.5)


@pytest.mark.parametrize("name", [n for n in tabular.AGENT_NAMES if n != "td-zero"])
def test_tabular_agents_solve_4x4(name):
    env = GridWorldEnv(size=4)
    agent = tabular.AGENTS[name](env, tabular.TabularConfig(seed=3))
    train_grid(env, agent, 512)
    ev = evaluate_grid(GridWorldEnv(size=4), agent, 16)
    assert ev.success_rate() == 1.0 and ev.mean_return() == pytest.approx(0.75, abs=0.05)


@pytest.mark.parametrize("name", planning.AGENT_NAMES)
def test_planning_agents_are_optimal_on_4x4(name):
    env = GridWorldEnv(size=4)
    agent = planning.AGENTS[name](env, planning.PlanningConfig())
    ev = evaluate_grid(env, agent, 4)
    assert ev.mean_return() == pytest.approx(0.75) and ev.mean_length() == 6 and ev.success_rate() == 1.0


def test_planning_on_8x8_with_traps_matches_published_return():
    start, goal = (0, 0), (7, 7)
    env = GridWorldEnv(size=8, traps=GridWorldEnv.generate_traps(8, 24, start, goal))
    for cls in (planning.ValueIterationAgent, planning.PolicyIterationAgent):
        ev = evaluate_grid(env, cls(env), 2)
        assert ev.mean_return() == pytest.approx(0.35)  # 13 steps at -0.05, then +1


def test_cartpole_physics_and_limits():
    env = CartPoleEnv()
    obs, _ = env.reset(seed=0)
    assert obs.shape == (4,) and np.all(np.abs(obs) <= 0.05)
    steps, term = 0, False
    while not term:
        obs, r, term, trunc, _ = env.step(1)  # always push right: falls quickly
        steps += 1
        assert r == 1.0
    assert 5 < steps < 60
    obs2, _ = env.reset(seed=0)
    assert np.allclose(obs2, CartPoleEnv().reset(seed=0)[0])


def test_ppo_bookkeeping_and_gae_numbers():
    agent = deep.PPOAgent(CartPoleEnv(), deep.DeepConfig(hidden_size=16, seed=24))
    obs, nxt = np.zeros(4, dtype=np.float32), np.ones(4, dtype=np.float32)
    a = agent.select_action(obs)
    agent.update(obs, a, 1.0, nxt, False, True)
    assert agent.pending_step is None and len(agent.rollout) == 1
    assert agent.rollout[0].log_prob.shape == torch.Size([]) and agent.rollout[0].value.shape == torch.Size([])
    agent = deep.PPOAgent(CartPoleEnv(), deep.DeepConfig(gamma=0.8, hidden_size=16), deep.PPOConfig(gae_lambda=0.5))

    def step(reward, terminated):
        return deep.RolloutStep(deep.Transition(obs, 0, reward, obs, terminated, False),
                                torch.as_tensor(0.0), torch.as_tensor(0.0))

    agent.rollout = [step(1.0, False), step(3.0, True)]
    assert agent._advantages(torch.as_tensor([0.5, 1.0])).tolist() == pytest.approx([2.1, 2.0])


@pytest.mark.parametrize("name", deep.AGENT_NAMES)
def test_deep_agents_train_and_evaluate(name):
    cfg = deep.DeepConfig(batch_size=4, warmup_steps=4, hidden_size=16, seed=24)
    env = CartPoleEnv()
    agent = deep.AGENTS[name](env, cfg)
    tr = train_control(env, agent, 16, seed=cfg.seed)
    ev = evaluate_control(CartPoleEnv(), agent, 4, seed=cfg.seed)
    assert tr.episodes[0].terminated or tr.episodes[0].truncated
    assert ev.mean_return() >= 8
    assert ev.termination_rate() + ev.success_rate() == 1.0


def test_cli_smoke(capsys, tmp_path):
    from zero_to_hero_b200.rl.cli import main
    main(["tabular", "render", "--size", "4"])
    assert "G" in capsys.readouterr().out
    main(["tabular", "train", "--size", "4", "--algorithm", "q-learning", "--train-episodes", "64",
          "--eval-episodes", "4", "--show-policy", "--plot", str(tmp_path / "c.png")])
    out = capsys.readouterr().out
    assert "eval mean return" in out and "saved to" in out
    main(["planning", "benchmark", "--size", "4", "--runs", "2", "--train-episodes", "2", "--eval-episodes", "2"])
    assert "value-iteration" in capsys.readouterr().out
