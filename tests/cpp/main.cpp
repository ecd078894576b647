#include "mini_test.hpp"

int main(int argc, char** argv) { return mini::runAll(argc, argv); }
