"""Model analysis: per-parameter statistics, entropy / top-2-gap histograms, log-probability visualisations."""
from .entropy import cb_compute_entropies, cb_compute_top2_gap, compute_entropy_histogram, compute_top2_gap_histogram  # noqa: F401
from .tree_stats import summary_statistics_for_tree  # noqa: F401
from .visualization import cb_compute_and_visualize_log_probs, visualize_log_prob_diff, visualize_log_probs  # noqa: F401
