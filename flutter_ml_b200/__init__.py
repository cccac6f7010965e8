"""B200-native compute backend for the flutter_ml autograd framework."""
