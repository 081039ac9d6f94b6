"""Character-level name models ("makemore"): bigram counts, bigram networks, MLP with batch
norm (raw tensors and a hand-rolled module system), manual back-propagation, a WaveNet-style
hierarchical model. Library counterparts of the reference's nn/makemore/*.py scripts."""
