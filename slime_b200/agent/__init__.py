"""Agent layer: chat-protocol adapters in front of the rollout engine, session trajectories, sandboxes, harness glue."""
