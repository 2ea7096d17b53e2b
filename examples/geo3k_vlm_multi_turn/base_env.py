"""Contract of an interaction environment for multi-turn rollouts.

``reset() -> (observation, info)`` once per episode, ``step(response_text) -> (observation, done, info)`` after every
assistant turn, ``close()`` at the end. An observation is a dict: ``obs_str`` (text shown to the model), optionally
``multi_modal_data`` (``{"image": [PIL images]}``) and a ``role``. ``format_observation`` turns it into the chat message
that is rendered and appended to the conversation. A module named by ``rollout_interaction_env_path`` exposes
``build_env(sample=..., args=...)``. (Same protocol as examples/geo3k_vlm_multi_turn/base_env.py in the reference.)
"""

from __future__ import annotations


class BaseInteractionEnv:
    def reset(self):
        raise NotImplementedError

    def step(self, response_text: str):
        raise NotImplementedError

    def close(self):
        pass

    def format_observation(self, observation: dict | None) -> dict:
        observation = observation or {}
        content = [{"type": "image", "image": im} for ims in (observation.get("multi_modal_data") or {}).values() for im in ims]
        content.append({"type": "text", "text": observation.get("obs_str", "")})
        return {"role": "user", "content": content}
