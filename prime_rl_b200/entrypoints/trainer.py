"""``trainer @ trainer.toml`` (normally under ``torchrun``): the RL trainer process."""

from ..trainer.rl.train import main

if __name__ == "__main__":
    main()
