/* Empty stand-in: the archive writer header includes this protobuf header but uses nothing from it. */
