"""A unit of queued work: one prompt plus its generation settings.  Ordering is by cost
(prompt length + tokens to generate) so that cheap requests batch first (reference:
metaseq/service/workers.py:26-62)."""
from __future__ import annotations

import queue
from dataclasses import dataclass, field
from typing import Any

from .queue import PriorityQueueRingShard, PriorityQueueRingShardKeyable


@dataclass
class WorkItem(PriorityQueueRingShardKeyable):
    cost: int
    uid: int
    return_queue: Any
    data: Any
    prompt_len: int = 0
    gen_len: int = 0

    def __lt__(self, other):
        return (self.cost, self.uid) < (other.cost, other.uid)

    def __eq__(self, other):
        return isinstance(other, WorkItem) and self.uid == other.uid and self.cost == other.cost

    def queue_key(self):
        # requests can share a batch only when every sampling parameter matches
        d = {k: v for k, v in self.data.items() if k not in ("input", "seed", "min_tokens", "max_tokens")}
        d = {k: (tuple(v) if isinstance(v, list) else v) for k, v in d.items()}
        return PriorityQueueRingShard.key_from_dict(d)

    @staticmethod
    def generate_worker(encoded_prompt, batch_queue, **generation_args):
        """Queues one prompt and blocks until its result comes back.  The cost grows with the prompt length
        linearly (feed-forward work) plus quadratically (attention), so long prompts sort behind short ones
        (reference: metaseq/service/workers.py:52-62)."""
        import math

        answer = queue.Queue()
        n = len(encoded_prompt)
        cost = n + int(math.ceil((n / 10) ** 2))
        batch_queue.put(WorkItem(cost, 0, answer, {"input": encoded_prompt, **generation_args}))
        _, result = answer.get()
        return result
