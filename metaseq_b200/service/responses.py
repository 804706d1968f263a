"""OpenAI-style response envelope (reference: metaseq/service/responses.py:13-38)."""
from __future__ import annotations

import time
import uuid


class OAIResponse:
    def __init__(self, results: list) -> None:
        self.results = results
        self.response_id = str(uuid.uuid4())
        self.created = int(time.time())

    def __dict__(self):
        return {
            "id": self.response_id,
            "object": "text_completion",
            "created": self.created,
            "model": "/".join(("metaseq_b200", "opt")),
            "choices": [
                {
                    "text": r["text"],
                    "logprobs": {
                        "tokens": r["tokens"],
                        "token_logprobs": r["token_scores"],
                        "text_offset": r["text_offset"],
                        "top_logprobs": r["top_logprobs"],
                        "finish_reason": "length",
                    },
                }
                for r in self.results
            ],
        }

    def to_dict(self):
        return self.__dict__()
