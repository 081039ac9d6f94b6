"""Learning-curve plot: rolling-mean return per agent, mean ± std over runs (rl/common/plot.py of
the reference). Uses matplotlib's headless Agg backend when matplotlib is installed; without it
the same curves are written as CSV next to the requested path."""
from __future__ import annotations

from pathlib import Path

import numpy as np


def rolling_mean(values: np.ndarray, window: int) -> np.ndarray:
    if window <= 1 or len(values) < window:
        return values
    return np.convolve(values, np.ones(window) / window, mode="valid")


def curves(run_groups, rolling_window: int = 16):
    """[(agent_name, episodes, mean, std)] for each group of runs of one agent."""
    out = []
    for runs in run_groups:
        smoothed = np.stack([rolling_mean(r.returns(), rolling_window) for r in runs])
        mean, std = smoothed.mean(axis=0), smoothed.std(axis=0)
        offset = len(runs[0].returns()) - len(mean)
        out.append((runs[0].agent_name, np.arange(offset, offset + len(mean)), mean, std))
    return out


def plot_returns(run_groups, output_path, rolling_window: int = 16) -> Path:
    output_path = Path(output_path)
    output_path.parent.mkdir(parents=True, exist_ok=True)
    data = curves(run_groups, rolling_window)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        csv = output_path.with_suffix(".csv")
        with open(csv, "w") as f:
            f.write("agent,episode,mean,std\n")
            for name, ep, mean, std in data:
                for e, m, s in zip(ep, mean, std):
                    f.write(f"{name},{e},{m:.6f},{s:.6f}\n")
        return csv
    fig, ax = plt.subplots(figsize=(10, 5))
    if sum(len(r) for r in run_groups) == 1:
        ax.plot(run_groups[0][0].returns(), alpha=0.2)
    for name, ep, mean, std in data:
        ax.plot(ep, mean, label=name)
        ax.fill_between(ep, mean - std, mean + std, alpha=0.2)
    ax.set_xlabel("episode")
    ax.set_ylabel(f"episode return, {rolling_window}-episode rolling mean")
    ax.legend()
    ax.grid(alpha=0.25)
    fig.tight_layout()
    fig.savefig(output_path, dpi=160)
    plt.close(fig)
    return output_path
