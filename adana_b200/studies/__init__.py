"""Scaling studies: from a table of finished runs to the numbers and figures of the optimizer comparison.

  runs        the run table (local experiment folders or a W&B project), disk cache, shared selections
  sizes       parameter counts per scaling rule, compute formulas, Chinchilla budgets
  lr_law      top-K learning rates per size -> lr*(P) = a (b + P)^d, bootstrap intervals
  curvature   parabola of loss in log lr per size, cost of a mis-set learning rate
  loss_laws   loss against compute: single / broken power laws, joint fits with a shared floor, compute multiplier
  savings     compute saved against a baseline, measured and propagated through lr uncertainty
  gamma3      best long-momentum multiplier against the length of training
  tau_cdf     tau distributions rebuilt from the stored order statistics
  sweeps      best run per size, GPU-hours ledger, logged optimizer statistics, Hoyer and kappa sweeps
  palette     one colour / line style / legend name per optimizer
  panels      SVG drawings of all of the above

    python -m adana_b200.studies --help
"""
