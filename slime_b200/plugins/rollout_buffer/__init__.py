"""Stand-alone trajectory buffer: generators write finished trajectories over HTTP, the trainer reads whole groups."""
