"""longbow-quarrel_b200: a small, whole model library for the Llama 3 dense decoder
(the Fetorax decoder of attention, retention and mLSTM layers, the Zoporax decoder of latent attention, lightning layers and routed experts, and the Raritar and Lavutar decoders) on one B200 -- configuration, weights, layers from parts, a paged cache with a slot
per sequence, one step function, generation and sampling, trace replay -- on
hand-written sm_100a kernels."""
__version__ = "0.1.0"
