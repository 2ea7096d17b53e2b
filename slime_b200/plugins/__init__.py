"""Optional pieces that sit beside the core framework: the stand-alone rollout buffer service, model plug-ins."""
