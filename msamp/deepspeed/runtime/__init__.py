"""Engine, configuration and optimizers behind ``msamp.deepspeed``."""
