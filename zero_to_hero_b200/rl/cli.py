"""Command line for the RL code: `python -m zero_to_hero_b200.rl.cli <family> <command>`.

    ... tabular  render | train --algorithm q-learning [--show-policy] | benchmark --runs 8
    ... planning render | train --algorithm mcts | benchmark
    ... deep     train --algorithm ppo | benchmark --runs 8

Same sub-commands and defaults as rl/common/grid_cli.py, rl/tabular/cli.py, rl/planning/cli.py
and rl/deep/cli.py of the reference (8x8 grid, env seed 24, 512 training / 32 evaluation
episodes, benchmark over `--runs` seed pairs printing mean ± std per agent, optional plot).
"""
from __future__ import annotations

import argparse
from dataclasses import replace

import numpy as np

from . import deep, planning, tabular
from .core import evaluate_control, evaluate_grid, spawn_seeds, train_control, train_grid
from .envs import CartPoleEnv, GridWorldEnv
from .plot import plot_returns


def make_grid(size: int, env_seed: int) -> GridWorldEnv:
    start, goal = (0, 0), (size - 1, size - 1)
    return GridWorldEnv(size=size, start=start, traps=GridWorldEnv.generate_traps(size, env_seed, start, goal))


def mean_std(results, metric: str, percent: bool = False) -> str:
    v = np.array([getattr(r, metric)() for r in results])
    k, suffix = (100.0, "%") if percent else (1.0, "")
    return f"{np.mean(v) * k:.1f} ± {np.std(v) * k:.1f}{suffix}"


def _family(name: str):
    if name == "tabular":
        return tabular.AGENTS, tabular.TabularConfig, True
    if name == "planning":
        return planning.AGENTS, planning.PlanningConfig, True
    return deep.AGENTS, deep.DeepConfig, False


def run_one(family: str, algorithm: str, a, env_seed: int, agent_seed: int):
    agents, cfg_cls, is_grid = _family(family)
    cfg = replace(cfg_cls(), seed=agent_seed)
    if is_grid:
        env = make_grid(a.size, env_seed)
        agent = agents[algorithm](env, cfg)
        tr = train_grid(env, agent, a.train_episodes)
        ev = evaluate_grid(make_grid(a.size, env_seed), agent, a.eval_episodes)
        return agent, env, tr, ev
    env = CartPoleEnv()
    agent = agents[algorithm](env, cfg)
    tr = train_control(env, agent, a.train_episodes, seed=agent_seed)
    ev = evaluate_control(CartPoleEnv(), agent, a.eval_episodes, seed=agent_seed)
    return agent, env, tr, ev


def cmd_render(family, a):
    env = make_grid(a.size, a.env_seed)
    env.reset()
    print(env.render())


def cmd_train(family, a):
    agent, env, tr, ev = run_one(family, a.algorithm, a, a.env_seed, a.agent_seed)
    print(f"trained {tr.agent_name} for {len(tr.episodes)} episodes")
    print(f"train success rate: {tr.success_rate():.2%}")
    print(f"eval mean return: {ev.mean_return():.3f}")
    print(f"eval success rate: {ev.success_rate():.2%}")
    if a.plot:
        print(f"learning curves plot saved to {plot_returns([[tr]], a.plot)}")
    if getattr(a, "show_policy", False) and hasattr(agent, "q_values"):
        print(env.render_policy(agent.q_values))


def cmd_benchmark(family, a):
    agents, _, _ = _family(family)
    seeds = spawn_seeds(a.seed, a.runs)
    print(f"{'run':>3}  {'env_seed':>10}  {'agent_seed':>10}")
    for i, (e, g) in enumerate(seeds):
        print(f"{i:>3}  {e:>10}  {g:>10}")
    row = "{:<16}  {:>13}  {:>14}  {:>14}"
    print()
    print(row.format("agent", "mean_return", "success", "mean_len"))
    groups = []
    for name in agents:
        trs, evs = [], []
        for e, g in seeds:
            _, _, tr, ev = run_one(family, name, a, e, g)
            trs.append(tr)
            evs.append(ev)
        groups.append(trs)
        print(row.format(name, mean_std(evs, "mean_return"), mean_std(evs, "success_rate", True),
                         mean_std(evs, "mean_length")))
    if a.plot:
        print(f"learning curves plot saved to {plot_returns(groups, a.plot)}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="zero_to_hero_b200.rl.cli")
    fam = ap.add_subparsers(dest="family", required=True)
    for family in ("tabular", "planning", "deep"):
        agents, _, is_grid = _family(family)
        fp = fam.add_parser(family)
        sub = fp.add_subparsers(dest="command", required=True)
        cmds = (["render"] if is_grid else []) + ["train", "benchmark"]
        for c in cmds:
            p = sub.add_parser(c)
            if is_grid:
                p.add_argument("--size", type=int, default=8)
                p.add_argument("--env-seed", type=int, default=24)
            else:
                p.set_defaults(size=0, env_seed=0)
            if c != "render":
                p.add_argument("--train-episodes", type=int, default=512)
                p.add_argument("--eval-episodes", type=int, default=32)
                p.add_argument("--plot", default="")
            if c == "train":
                p.add_argument("--algorithm", choices=list(agents), default=list(agents)[-1])
                p.add_argument("--agent-seed", type=int, default=0 if is_grid else 24)
                if family == "tabular":
                    p.add_argument("--show-policy", action="store_true")
            if c == "benchmark":
                p.add_argument("--runs", type=int, default=8)
                p.add_argument("--seed", type=int, default=24)
    return ap


def main(argv=None):
    a = build_parser().parse_args(argv)
    {"render": cmd_render, "train": cmd_train, "benchmark": cmd_benchmark}[a.command](a.family, a)


if __name__ == "__main__":
    main()
