"""``python -m mintext.train``: the training CLI under the reference's module path (mintext/train.py)."""

from mintext_b200.train import *  # noqa: F401,F403
from mintext_b200.train import main, setup_training, train  # noqa: F401

if __name__ == "__main__":
    main()
