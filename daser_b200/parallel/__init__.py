"""Multi-process arrangements: tensor parallelism over peer memory, pipeline stages, peer liveness."""
