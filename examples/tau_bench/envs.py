"""Environments for the tool-agent example.

``make_env(name, task_index)`` returns an object with

    tools        list of OpenAI-style function schemas
    system       str, the policy / wiki text shown to the agent
    reset()   -> first user message (str)
    step(action) -> (observation str, reward float, done bool); ``action`` is {"name": tool name, "arguments": {...}} or
                    {"name": "respond", "arguments": {"content": text}} for a message to the simulated user

``retail`` / ``airline`` come from the ``tau_bench`` package when it is installed (its user simulator needs an LLM API
key); ``mock_retail`` is a small self-contained stand-in with a scripted user, a two-table database and a reward that
compares the final database with the task's goal, so that the example and its tests run anywhere. Same role as
examples/tau-bench/tau1_mock.py and the ``tau_bench.envs.get_env`` call of generate_with_tau.py in the reference.
"""

from __future__ import annotations

import copy
import json

_FN = lambda name, desc, **props: {"type": "function", "function": {  # noqa: E731
    "name": name, "description": desc,
    "parameters": {"type": "object", "properties": {k: {"type": v} for k, v in props.items()}, "required": list(props)}}}

MOCK_TASKS = [
    {"user": "Hi, I'd like to cancel my order #W100, I ordered it by mistake.", "goal": {"W100": "cancelled"},
     "follow_up": "Yes, please go ahead. That is all, thanks."},
    {"user": "Can you change the shipping address of order #W200 to 12 Elm Street?", "goal": {"W200": "pending"},
     "goal_address": {"W200": "12 Elm Street"}, "follow_up": "Yes, confirmed. Nothing else."},
    {"user": "What is the status of order #W300?", "goal": {"W300": "delivered"}, "follow_up": "Thanks, bye."},
]
_DB = {"W100": {"status": "pending", "address": "1 Main St"}, "W200": {"status": "pending", "address": "9 Oak Ave"},
       "W300": {"status": "delivered", "address": "4 Pine Rd"}}  # fmt: skip


class MockRetailEnv:
    system = ("You are a retail support agent. Look an order up before acting on it. Ask the user to confirm before you "
              "cancel or modify an order. Delivered orders cannot be changed. End the conversation when the user is done.")  # fmt: skip
    tools = [_FN("get_order", "Look up an order.", order_id="string"),
             _FN("cancel_order", "Cancel a pending order.", order_id="string"),
             _FN("set_address", "Change the shipping address of a pending order.", order_id="string", address="string")]  # fmt: skip

    def __init__(self, task_index: int = 0, max_steps: int = 12):
        self.task = MOCK_TASKS[task_index % len(MOCK_TASKS)]
        self.max_steps = max_steps

    def reset(self) -> str:
        self.db, self.steps, self.user_turns = copy.deepcopy(_DB), 0, 0
        return self.task["user"]

    def _reward(self) -> float:
        ok = all(self.db[o]["status"] == s for o, s in self.task["goal"].items())
        ok &= all(self.db[o]["address"] == a for o, a in self.task.get("goal_address", {}).items())
        untouched = all(self.db[o] == _DB[o] for o in _DB if o not in self.task["goal"])
        return float(ok and untouched)

    def step(self, action: dict):
        self.steps += 1
        name, a = action.get("name"), action.get("arguments") or {}
        if name == "respond":
            self.user_turns += 1
            if self.user_turns == 1:
                return self.task["follow_up"], 0.0, False
            return "###STOP###", self._reward(), True
        order = self.db.get(str(a.get("order_id", "")).lstrip("#"))
        if name == "get_order":
            obs = json.dumps(order) if order else "Error: order not found"
        elif name in ("cancel_order", "set_address"):
            if order is None:
                obs = "Error: order not found"
            elif order["status"] != "pending":
                obs = "Error: only pending orders can be changed"
            elif name == "cancel_order":
                order["status"] = "cancelled"
                obs = "Order cancelled"
            else:
                order["address"] = str(a.get("address", ""))
                obs = "Address updated"
        else:
            obs = f"Error: unknown tool {name}"
        done = self.steps >= self.max_steps
        return obs, (self._reward() if done else 0.0), done


class TauBenchEnv:
    """Adapter over ``tau_bench.envs.get_env`` (retail / airline)."""

    def __init__(self, name: str, task_index: int, user_strategy: str = "llm", user_model: str = "gpt-4o", user_provider: str = "openai",
                 task_split: str = "train"):  # fmt: skip
        from tau_bench.envs import get_env

        self.env = get_env(name, user_strategy=user_strategy, user_model=user_model, user_provider=user_provider,
                           task_split=task_split, task_index=task_index)  # fmt: skip
        self.task_index = task_index
        self.tools, self.system = self.env.tools_info, self.env.wiki

    def reset(self) -> str:
        return self.env.reset(task_index=self.task_index).observation

    def step(self, action: dict):
        from tau_bench.types import Action

        kw = action.get("arguments") or {}
        r = self.env.step(Action(name=action["name"], kwargs=kw))
        return r.observation, float(r.reward), bool(r.done)


def make_env(name: str, task_index: int, **kw):
    if name == "mock_retail":
        return MockRetailEnv(task_index)
    return TauBenchEnv(name, task_index, **kw)
