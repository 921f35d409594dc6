class Encoding:
    def __init__(self, name: str = "gpt2") -> None:
        self.name = name
        self.n_vocab = 50257
        self.eot_token = 50256

    def encode(self, text, allowed_special=None):
        return list(text.encode("utf-8"))

    encode_ordinary = encode

    def decode(self, ids):
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")
