"""``rstorch.data``: Dataset, DataLoader and samplers."""
from torsh_b200.data import *  # noqa: F401,F403
from torsh_b200.data import DataLoader, Dataset, DistributedSampler, TensorDataset  # noqa: F401
