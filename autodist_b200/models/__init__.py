"""Model families of the reference's examples and benchmarks: BERT pre-training, ImageNet CNNs (ResNet-101, VGG-16,
DenseNet-121, Inception-style), the LM1B LSTM language model, NeuMF and the small getting-started models."""
