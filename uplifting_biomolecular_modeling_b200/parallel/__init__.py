"""Multi-GPU machinery: layouts, the communication surface, symmetric peer memory, the row-sharded pair
stack (``big --n_gpu P``), tensor parallelism for the sequence models, launcher and checkpoints."""
