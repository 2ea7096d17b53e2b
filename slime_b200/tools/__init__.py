"""Command-line tools: checkpoint converters, rollout profiling, trace analysis. Run as ``python -m slime_b200.tools.<name>``."""
