"""OpenAI-style response envelope (reference: metaseq/service/responses.py:13-38)."""
from __future__ import annotations

import time
import uuid

MODEL_NAME = "metaseq_b200/opt"


def _choice(result: dict) -> dict:
    logprobs = {"tokens": result["tokens"], "token_logprobs": result["token_scores"],
                "text_offset": result["text_offset"], "top_logprobs": result["top_logprobs"],
                "finish_reason": "length"}
    return {"text": result["text"], "logprobs": logprobs}


class OAIResponse:
    """One ``text_completion`` object for a list of generation results."""

    def __init__(self, results: list) -> None:
        self.results = results
        self.created = int(time.time())
        self.response_id = str(uuid.uuid4())

    def to_dict(self):
        return {"id": self.response_id, "object": "text_completion", "created": self.created, "model": MODEL_NAME,
                "choices": [_choice(r) for r in self.results]}

    def __dict__(self):
        return self.to_dict()
