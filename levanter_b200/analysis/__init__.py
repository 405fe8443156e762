from .tree_stats import summary_statistics_for_tree  # noqa: F401
