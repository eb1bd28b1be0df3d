"""Model registry (utils/fullgraph_sp_support.py:778-805 in the reference, plus NAGphormer)."""
from .exphormer import Exphormer
from .graphgps import GraphGPS
from .graphormer import Graphormer
from .gt import GT
from .nagphormer import NAGphormer

MODEL_REGISTRY = {"graphormer": Graphormer, "gt": GT, "graphgps": GraphGPS, "exphormer": Exphormer,
                  "nagphormer": NAGphormer}

__all__ = ["Graphormer", "GT", "GraphGPS", "Exphormer", "NAGphormer", "MODEL_REGISTRY"]
