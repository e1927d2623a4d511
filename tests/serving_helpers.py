"""Helpers shared by the serving tests (module level so that a spawned coordinator process can unpickle them)."""
import socket


class CharTokenizer:
    """tokenize: one id per character; detokenize: the ids joined by commas."""

    bos = 1

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size

    def tokenize(self, text):
        return [ord(c) % self.vocab_size for c in text]

    def detokenize(self, tokens):
        return ",".join(str(t) for t in tokens)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
