"""Reinforcement learning: GridWorld / CartPole environments, tabular, planning and deep agents."""
