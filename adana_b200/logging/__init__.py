"""Observability: optimizer-schedule logs, tau statistics, training-dynamics logger, MoE routing plots."""
