import enum


class Format(enum.Enum):
    E4M3 = "e4m3"
    HYBRID = "hybrid"


class Float8BlockScaling:
    def __init__(self, **kwargs) -> None:
        self.kwargs = kwargs
